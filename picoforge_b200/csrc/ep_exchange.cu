// Packing and unpacking of the expert-parallel exchange messages.
//
// A rank sends every (token, slot) pair to the rank that owns the pair's expert.  The message a rank
// sends has `world` blocks of `cap` row slots; a slot is `pitch` floats: the token's `hidden` activations, then
// one word with the expert's index inside the destination's shard (0xffffffff: slot unused), then padding to
// a multiple of four words.  One all-to-all moves rows and ids together.
//
//   ep_plan_kernel      one CTA: destination and stable position of every pair (pairs keep their order inside
//                       a block, so the destination sees each source's rows in pair order), id words written,
//                       unused slots marked
//   ep_scatter_kernel   one CTA per pair: the token's row into its slot
//   ep_ids_kernel       receiver: the id words of all slots into a contiguous array for the dispatch
//   ep_gather_kernel    source, after the return all-to-all: slot -> pair order for the combine
#include <cuda_runtime.h>
#include <stdint.h>

#include "cuda_shim.h"

namespace qw4 {

constexpr uint32_t EP_MAX_WORLD = 64;

__global__ void __launch_bounds__(1024) ep_plan_kernel(const uint32_t *__restrict__ ids, uint32_t pairs, uint32_t experts_per_rank, uint32_t world,
                                                       uint32_t cap, float *__restrict__ msg, uint32_t pitch, uint32_t hidden,
                                                       uint32_t *__restrict__ slot_of_pair, uint32_t *status) {
    __shared__ uint32_t base[EP_MAX_WORLD];                  // rows placed so far, per destination
    __shared__ uint32_t wcount[32][EP_MAX_WORLD];            // this batch of 1024 pairs: rows of each warp per destination, then their first position
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    uint32_t *words = reinterpret_cast<uint32_t *>(msg);
    for (uint32_t s = tid; s < world * cap; s += 1024) words[(uint64_t)s * pitch + hidden] = 0xffffffffu;
    if (tid < EP_MAX_WORLD) base[tid] = 0;
    __syncthreads();
    for (uint32_t first = 0; first < pairs; first += 1024) {
        const uint32_t p = first + tid;
        const uint32_t id = p < pairs ? ids[p] : 0xffffffffu;
        const uint32_t dest = id / experts_per_rank;
        const bool ok = p < pairs && dest < world;
        for (uint32_t i = tid; i < 32 * EP_MAX_WORLD; i += 1024) (&wcount[0][0])[i] = 0;
        __syncthreads();
        const uint32_t same = __match_any_sync(0xffffffffu, ok ? dest : 0xffffffffu);
        const uint32_t rank = __popc(same & ((1u << lane) - 1u));
        if (ok && rank == 0) wcount[warp][dest] = __popc(same);
        __syncthreads();
        if (tid < world) {
            uint32_t run = base[tid];
            for (uint32_t w = 0; w < 32; w++) { const uint32_t c = wcount[w][tid]; wcount[w][tid] = run; run += c; }
            base[tid] = run;
        }
        __syncthreads();
        if (p < pairs) {
            uint32_t slot = 0xffffffffu;
            if (ok) {
                const uint32_t pos = wcount[warp][dest] + rank;
                if (pos < cap) {
                    slot = dest * cap + pos;
                    words[(uint64_t)slot * pitch + hidden] = id - dest * experts_per_rank;
                }
            }
            if (slot == 0xffffffffu) atomicOr(status, QW4SH_ERR_BOUNDS);
            slot_of_pair[p] = slot;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(128) ep_scatter_kernel(const float *__restrict__ x, uint32_t k, uint32_t hidden, const uint32_t *__restrict__ slot_of_pair,
                                                         float *__restrict__ msg, uint32_t pitch) {
    const uint32_t p = blockIdx.x, slot = slot_of_pair[p];
    if (slot == 0xffffffffu) return;
    const float4 *src = reinterpret_cast<const float4 *>(x + (uint64_t)(p / k) * hidden);
    float4 *dst = reinterpret_cast<float4 *>(msg + (uint64_t)slot * pitch);
    for (uint32_t i = threadIdx.x; i < hidden / 4; i += 128) dst[i] = src[i];
}

__global__ void ep_ids_kernel(const float *__restrict__ msg, uint32_t pitch, uint32_t hidden, uint32_t rows, uint32_t *__restrict__ ids) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) ids[r] = reinterpret_cast<const uint32_t *>(msg)[(uint64_t)r * pitch + hidden];
}

__global__ void __launch_bounds__(128) ep_gather_kernel(const float *__restrict__ back, uint32_t hidden, const uint32_t *__restrict__ slot_of_pair,
                                                        float *__restrict__ pair_out) {
    const uint32_t p = blockIdx.x, slot = slot_of_pair[p];
    float4 *dst = reinterpret_cast<float4 *>(pair_out + (uint64_t)p * hidden);
    if (slot == 0xffffffffu) {
        for (uint32_t i = threadIdx.x; i < hidden / 4; i += 128) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float4 *src = reinterpret_cast<const float4 *>(back + (uint64_t)slot * hidden);
    for (uint32_t i = threadIdx.x; i < hidden / 4; i += 128) dst[i] = src[i];
}

}  // namespace qw4

using namespace qw4;

extern "C" int qw4sh_note_launch(const char *name);

// Words per message slot for rows of `hidden` floats.
extern "C" uint32_t qw4sh_ep_pitch(uint32_t hidden) { return hidden + 4; }

extern "C" int qw4sh_ep_pack(const float *x, uint32_t tokens, uint32_t k, uint32_t hidden, const uint32_t *ids, uint32_t experts_per_rank,
                             uint32_t world, uint32_t cap, float *msg, uint32_t *slot_of_pair, uint32_t *status, void *stream) {
    if (!tokens) return 0;
    if (world > EP_MAX_WORLD || hidden % 4 || !experts_per_rank) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t pitch = qw4sh_ep_pitch(hidden);
    ep_plan_kernel<<<1, 1024, 0, s>>>(ids, tokens * k, experts_per_rank, world, cap, msg, pitch, hidden, slot_of_pair, status);
    int rc = qw4sh_note_launch("ep_plan_kernel");
    if (rc) return rc;
    ep_scatter_kernel<<<tokens * k, 128, 0, s>>>(x, k, hidden, slot_of_pair, msg, pitch);
    return qw4sh_note_launch("ep_scatter_kernel");
}

extern "C" int qw4sh_ep_ids(const float *msg, uint32_t hidden, uint32_t rows, uint32_t *ids, void *stream) {
    if (!rows) return 0;
    ep_ids_kernel<<<(rows + 255) / 256, 256, 0, (cudaStream_t)stream>>>(msg, qw4sh_ep_pitch(hidden), hidden, rows, ids);
    return qw4sh_note_launch("ep_ids_kernel");
}

extern "C" int qw4sh_ep_gather(const float *back, uint32_t hidden, const uint32_t *slot_of_pair, uint32_t pairs, float *pair_out, void *stream) {
    if (!pairs) return 0;
    ep_gather_kernel<<<pairs, 128, 0, (cudaStream_t)stream>>>(back, hidden, slot_of_pair, pair_out);
    return qw4sh_note_launch("ep_gather_kernel");
}
