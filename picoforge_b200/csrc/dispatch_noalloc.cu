// Dispatch lists without any allocation.
//
// qw4cu_group_pairs_device_noalloc builds the same per-expert pair lists as
// qw4_moe_group_pairs, for ids that already sit in device memory, and allocates nothing: not
// with cudaMalloc, not through a stream or event it would have to create, not on the host.
// It exists for callers that must not allocate while they run: a decode loop that has already
// handed every spare byte of HBM to weights and caches, where an allocation can fail and
// cudaMalloc also stalls the whole device while it runs.
//
// The kernel's working memory (per-expert counters and cursors, the list of non-empty experts
// and an error word) lives in the file-scope __device__ array below.  Every GPU that loads this
// library holds those 33 KB until the process exits.  All calls on a device share the array and
// it keeps what the previous call left in it, so the kernel clears what it needs first, and two
// calls that overlap on the GPU (from two host threads or two streams, say) would race: callers
// serialise.
//
// Stream: the call enqueues on the stream the rest of the library uses at that moment (the one
// given to qw4cu_set_stream, else the library's own stream if a workspace has already created
// it, else the legacy default stream), so ids written by an earlier library call on that stream
// are ordered before it; it then waits for that stream and returns the kernel's verdict.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/qwen4_moe_b200.h"
#include "cuda_shim.h"

#define NOALLOC_MAX_EXPERTS QW4CU_NOALLOC_MAX_EXPERTS
#define NOALLOC_THREADS 1024

// [0, E]            counters, then exclusive offsets / cursors
// [E+1, 2E+1]       non-empty expert list (count first)
// [2E+2, 2E+9]      error word and spare
static __device__ __align__(256) uint32_t g_dispatch_scratch[2 * (NOALLOC_MAX_EXPERTS + 1) + 8];

// In host code the array's name is only a stand-in: the device address is fetched once per
// device with cudaGetSymbolAddress and that pointer is what the kernel receives.
static uint32_t *g_scratch_address[64] = {nullptr};

extern "C" int qw4sh_note_launch(const char *name);

// One CTA.  Histogram, serial prefix, then a stable scatter: every thread walks ALL pairs in
// ascending order (the whole CTA reads the same word at the same time, one broadcast load) and
// the thread that owns the pair's expert (expert % threads) hands out that expert's next row
// from its cursor.  A cursor has one owner, so no atomics and the order inside an expert is the
// pair order.  Cost: `pairs` loop steps per thread, whatever the expert count.
__global__ void __launch_bounds__(NOALLOC_THREADS) group_noalloc_kernel(uint32_t experts, uint32_t pairs, const uint32_t *__restrict__ ids,
                                                                        uint32_t *__restrict__ offsets, uint32_t *__restrict__ pair_to_row,
                                                                        uint32_t *__restrict__ row_to_pair, uint32_t *scratch) {
    uint32_t *counts = scratch, *active = scratch + experts + 1, *status = scratch + 2 * (experts + 1);
    for (uint32_t e = threadIdx.x; e <= experts; e += blockDim.x) { counts[e] = 0; active[e] = 0; }
    if (threadIdx.x < 8) status[threadIdx.x] = 0;            // the array still holds the last call's values
    __syncthreads();
    bool bad = false;
    for (uint32_t p = threadIdx.x; p < pairs; p += blockDim.x) {
        const uint32_t e = ids[p];
        if (e < experts) atomicAdd(&counts[e], 1u); else bad = true;
    }
    if (bad) atomicOr(status, 2u);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t running = 0, n_active = 0;
        for (uint32_t e = 0; e < experts; e++) {
            const uint32_t c = counts[e];
            counts[e] = running; offsets[e] = running;
            if (c) active[1 + n_active++] = e;
            running += c;
        }
        counts[experts] = running; offsets[experts] = running; active[0] = n_active;
    }
    __syncthreads();
    const uint32_t me = threadIdx.x;
    uint32_t p = 0;
    for (; p + 4 <= pairs; p += 4) {                          // four loads in flight per step
        const uint32_t e0 = ids[p], e1 = ids[p + 1], e2 = ids[p + 2], e3 = ids[p + 3];
        if (e0 < experts && e0 % NOALLOC_THREADS == me) { const uint32_t r = counts[e0]++; pair_to_row[p] = r; row_to_pair[r] = p; }
        if (e1 < experts && e1 % NOALLOC_THREADS == me) { const uint32_t r = counts[e1]++; pair_to_row[p + 1] = r; row_to_pair[r] = p + 1; }
        if (e2 < experts && e2 % NOALLOC_THREADS == me) { const uint32_t r = counts[e2]++; pair_to_row[p + 2] = r; row_to_pair[r] = p + 2; }
        if (e3 < experts && e3 % NOALLOC_THREADS == me) { const uint32_t r = counts[e3]++; pair_to_row[p + 3] = r; row_to_pair[r] = p + 3; }
    }
    for (; p < pairs; p++) {
        const uint32_t e = ids[p];
        if (e < experts && e % NOALLOC_THREADS == me) { const uint32_t r = counts[e]++; pair_to_row[p] = r; row_to_pair[r] = p; }
    }
}

static Qwen4Status answer(Qwen4Error *err, Qwen4Status code, const char *detail) {
    if (err) {
        memset(err, 0, sizeof *err);
        err->code = code;
        if (code != QW4_OK) {
            snprintf(err->subject, sizeof err->subject, "qwen4_moe");
            snprintf(err->detail, sizeof err->detail, "%s", detail);
        }
    }
    return code;
}

extern "C" Qwen4Status qw4cu_group_pairs_device_noalloc(uint32_t experts, uint32_t top_k, size_t tokens, const uint32_t *ids_dev,
                                                        uint32_t *offsets_dev, uint32_t *pair_to_row_dev, uint32_t *row_to_pair_dev,
                                                        Qwen4Error *err) {
    if (!experts || !top_k || top_k > experts) return answer(err, QW4_RANGE, "invalid expert count or top_k");
    if (experts > NOALLOC_MAX_EXPERTS) {
        char text[160];
        snprintf(text, sizeof text, "%u experts exceed the %d the built-in scratch array holds", experts, NOALLOC_MAX_EXPERTS);
        return answer(err, QW4_CAPACITY, text);
    }
    if (tokens > QW4CU_NOALLOC_MAX_PAIRS / top_k) {
        char text[160];
        snprintf(text, sizeof text, "%zu tokens x %u exceed the limit of %d pairs per call", tokens, top_k, QW4CU_NOALLOC_MAX_PAIRS);
        return answer(err, QW4_CAPACITY, text);
    }
    if (!offsets_dev || (tokens && (!ids_dev || !pair_to_row_dev || !row_to_pair_dev)))
        return answer(err, QW4_INVALID_ARGUMENT, "null device pointer");
    int device = 0;
    cudaError_t rc = cudaGetDevice(&device);
    if (rc != cudaSuccess || device < 0 || device >= 64) return answer(err, QW4_GPU_ERROR, "no current CUDA device");
    if (!g_scratch_address[device]) {                        // once per device, with that device current
        uint32_t *address = nullptr;
        rc = cudaGetSymbolAddress((void **)&address, g_dispatch_scratch);
        if (rc != cudaSuccess || !address) return answer(err, QW4_GPU_ERROR, cudaGetErrorString(rc));
        g_scratch_address[device] = address;
    }
    uint32_t *scratch = g_scratch_address[device];
    void *stream_in_force = nullptr;
    if (qw4sh_existing_stream(&stream_in_force)) return answer(err, QW4_GPU_ERROR, "no current CUDA device");
    cudaStream_t stream = (cudaStream_t)stream_in_force;
    group_noalloc_kernel<<<1, NOALLOC_THREADS, 0, stream>>>(experts, (uint32_t)(tokens * top_k), ids_dev, offsets_dev, pair_to_row_dev,
                                                            row_to_pair_dev, scratch);
    if (qw4sh_note_launch("group_noalloc_kernel")) return answer(err, QW4_GPU_ERROR, "dispatch launch failed");
    uint32_t status = 0;
    rc = cudaMemcpyAsync(&status, scratch + 2 * (experts + 1), sizeof status, cudaMemcpyDeviceToHost, stream);
    if (rc == cudaSuccess) rc = cudaStreamSynchronize(stream);
    if (rc != cudaSuccess) return answer(err, QW4_GPU_ERROR, cudaGetErrorString(rc));
    if (status & 2u) return answer(err, QW4_RANGE, "expert ID out of range");
    return answer(err, QW4_OK, "");
}
