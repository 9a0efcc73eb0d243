// CUDA kernels of the Qwen4 MoE layer for sm_100a, and the C shim that launches them.
//
// Path (one launch each; picoforge src/qwen4_moe.c:334-382 is the CPU statement of the
// same sequence):
//   router_logits  x -> logits [T,E] and the shared-expert gate logit [T]
//   route          softmax, top-k, renormalise -> ids, weights [T,k]
//   group          stable per-expert pair lists (dispatch)
//   gate_up        act[pair] = silu(gate_e x) * (up_e x), weights dequantised in registers
//   down_reduce    y[t] = sum_s w[t,s] (down_e act[pair]) + sigmoid(slogit[t]) (sdown sact[t])
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "cuda_shim.h"
#include "formats.cuh"
#include "route.cuh"

using namespace qw4;

// ------------------------------------------------------------------------------------
// Bookkeeping
// ------------------------------------------------------------------------------------
static thread_local char g_error[256] = "";
static unsigned long long g_launches = 0;

static int fail(cudaError_t e, const char *where) {
    snprintf(g_error, sizeof g_error, "%s: %s", where, cudaGetErrorString(e));
    return (int)e ? (int)e : -1;
}
#define CU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail(e_, #call); } while (0)
// Names of the kernels launched since qw4sh_launch_log_begin (string literals; the first LOG_CAP are kept).
extern "C" int qw4sh_fail_text(const char *text) {
    snprintf(g_error, sizeof g_error, "%s", text);
    return -1;
}
static const unsigned LOG_CAP = 512;
static const char *g_log[LOG_CAP];
static unsigned g_log_n = LOG_CAP;                // full: logging off until the first begin
static inline void log_launch(const char *name) {
    __sync_fetch_and_add(&g_launches, 1ull);
    const unsigned at = g_log_n;
    if (at < LOG_CAP) { g_log[at] = name; g_log_n = at + 1; }
}
#define LAUNCHED(name) do { log_launch(name); cudaError_t e_ = cudaGetLastError(); \
    if (e_ != cudaSuccess) return fail(e_, name); } while (0)

extern "C" int qw4sh_note_launch(const char *name) {
    log_launch(name);
    cudaError_t e = cudaGetLastError();
    return e != cudaSuccess ? fail(e, name) : 0;
}
extern "C" void qw4sh_launch_log_begin(void) { g_log_n = 0; }
// Comma-separated names since the last begin, truncated to `cap` bytes; returns the number of launches logged.
extern "C" size_t qw4sh_launch_log(char *out, size_t cap) {
    size_t at = 0;
    const unsigned n = g_log_n < LOG_CAP ? g_log_n : LOG_CAP;
    for (unsigned i = 0; i < n && cap; i++) {
        for (const char *c = g_log[i]; *c && at + 2 < cap; c++) out[at++] = *c;
        if (i + 1 < n && at + 2 < cap) out[at++] = ',';
    }
    if (cap) out[at] = 0;
    return n;
}

static bool g_constants_ready[64] = {false};
static int ensure_constants() {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(cudaErrorInvalidDevice, "device index");
    g_constants_ready[device] = true;
    return 0;
}

extern "C" int qw4sh_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { fail(cudaGetLastError(), "cudaGetDeviceCount"); return -1; }
    return n;
}
extern "C" int qw4sh_set_device(int device) { CU(cudaSetDevice(device)); return ensure_constants(); }
extern "C" int qw4sh_current_device(void) { int device = -1; return cudaGetDevice(&device) == cudaSuccess ? device : -1; }
extern "C" const char *qw4sh_last_error(void) { return g_error; }
extern "C" uint64_t qw4sh_launch_count(void) { return g_launches; }

extern "C" void *qw4sh_malloc(size_t bytes) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) { fail(cudaGetLastError(), "cudaMalloc"); return nullptr; }
    return p;
}
extern "C" void qw4sh_free(void *p) { if (p) cudaFree(p); }
extern "C" void *qw4sh_host_alloc(size_t bytes) {
    void *p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) { fail(cudaGetLastError(), "cudaHostAlloc"); return nullptr; }
    return p;
}
extern "C" void qw4sh_host_free(void *p) { if (p) cudaFreeHost(p); }
extern "C" int qw4sh_memcpy(void *dst, const void *src, size_t bytes, int to_device) {
    if (bytes) CU(cudaMemcpy(dst, src, bytes, to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost));
    return 0;
}
extern "C" int qw4sh_memcpy2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch,
                                    size_t width, size_t rows, int to_device, void *stream) {
    if (width && rows)
        CU(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, rows,
                             to_device == 2 ? cudaMemcpyDeviceToDevice : to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                             (cudaStream_t)stream));
    return 0;
}
extern "C" int qw4sh_memset_async(void *dst, int value, size_t bytes, void *stream) {
    if (bytes) CU(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return 0;
}
static cudaStream_t g_stream[64] = {nullptr};
extern "C" int qw4sh_shared_stream(void **stream) {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(cudaErrorInvalidDevice, "device index");
    if (!g_stream[device]) CU(cudaStreamCreateWithFlags(&g_stream[device], cudaStreamNonBlocking));
    *stream = g_stream[device];
    return ensure_constants();
}
extern "C" int qw4sh_stream_sync(void *stream) { CU(cudaStreamSynchronize((cudaStream_t)stream)); return 0; }
extern "C" int qw4sh_device_sync(void) { CU(cudaDeviceSynchronize()); return 0; }
extern "C" int qw4sh_event_create(void **event) { cudaEvent_t e; CU(cudaEventCreate(&e)); *event = e; return 0; }
extern "C" void qw4sh_event_destroy(void *event) { if (event) cudaEventDestroy((cudaEvent_t)event); }
extern "C" int qw4sh_event_record(void *event, void *stream) { CU(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); return 0; }
extern "C" float qw4sh_event_elapsed_ms(void *begin, void *end) {
    float ms = -1.0f;
    if (cudaEventSynchronize((cudaEvent_t)end) != cudaSuccess ||
        cudaEventElapsedTime(&ms, (cudaEvent_t)begin, (cudaEvent_t)end) != cudaSuccess) { fail(cudaGetLastError(), "event elapsed"); return -1.0f; }
    return ms;
}

// Writes a buffer larger than the 126 MB L2 so that the next kernel reads HBM.
static void *g_flush[64] = {nullptr};
static const size_t FLUSH_BYTES = 256u << 20;
extern "C" int qw4sh_flush_l2(void) {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (!g_flush[device]) CU(cudaMalloc(&g_flush[device], FLUSH_BYTES));
    CU(cudaMemsetAsync(g_flush[device], 0x5a, FLUSH_BYTES, 0));
    CU(cudaDeviceSynchronize());
    return 0;
}

// ------------------------------------------------------------------------------------
// Upload + regroup into the resident layout (formats.cuh)
// ------------------------------------------------------------------------------------
__global__ void regroup_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, uint32_t type,
                               uint64_t blocks_per_matrix, uint64_t matrices, uint64_t nb) {
    const uint64_t total = blocks_per_matrix * matrices;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t matrix = i / blocks_per_matrix, block = i % blocks_per_matrix;
        if (type == T_Q2_K) {
            const uint8_t *b = src + i * 84u;
            uint8_t *base = dst + matrix * blocks_per_matrix * 84u;
            for (int j = 0; j < 64; j++) base[block * 64u + j] = b[16 + j];
            for (int j = 0; j < 16; j++) base[blocks_per_matrix * 64u + block * 16u + j] = b[j];
            for (int j = 0; j < 4; j++) base[blocks_per_matrix * 80u + block * 4u + j] = b[80 + j];
        } else {                                               // IQ2_XXS
            const uint8_t *b = src + i * 66u;
            uint8_t *base = dst + matrix * blocks_per_matrix * 66u;
            const uint64_t row = block / nb, first = row * nb * 8u, swz = iq2_swizzle((uint32_t)row, (uint32_t)nb);
            for (int j = 0; j < 64; j++)                       // group c of the row goes to position c ^ swizzle
                base[(first + ((((block % nb) * 8u + (j >> 3))) ^ swz)) * 8u + (j & 7)] = b[2 + j];
            base[blocks_per_matrix * 64u + block * 2u] = b[0];
            base[blocks_per_matrix * 64u + block * 2u + 1] = b[1];
        }
    }
}

extern "C" int qw4sh_upload_tensor(const void *host, size_t bytes, uint32_t type, size_t k_storage,
                                   size_t n_out, size_t n_experts, void **device) {
    *device = nullptr;
    if (ensure_constants()) return -1;
    void *image = nullptr;
    CU(cudaMalloc(&image, bytes ? bytes : 16));
    if (type == T_Q2_K || type == T_IQ2_XXS) {
        void *staging = nullptr;
        cudaError_t e = cudaMalloc(&staging, bytes ? bytes : 16);
        if (e != cudaSuccess) { cudaFree(image); return fail(e, "cudaMalloc staging"); }
        e = cudaMemcpy(staging, host, bytes, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) {
            const uint64_t per_matrix = (uint64_t)n_out * (k_storage / 256);
            regroup_kernel<<<1184, 256>>>((const uint8_t *)staging, (uint8_t *)image, type, per_matrix, n_experts, k_storage / 256);
            __sync_fetch_and_add(&g_launches, 1ull);
            e = cudaGetLastError();
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
        }
        cudaFree(staging);
        if (e != cudaSuccess) { cudaFree(image); return fail(e, "regroup"); }
    } else if (bytes) {
        cudaError_t e = cudaMemcpy(image, host, bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { cudaFree(image); return fail(e, "cudaMemcpy weights"); }
    }
    *device = image;
    return 0;
}

// ------------------------------------------------------------------------------------
// Exact decode probe
// ------------------------------------------------------------------------------------
__global__ void decode_rows_kernel(DevTensor t, uint32_t expert, uint32_t row0, uint32_t rows, float *out) {
    const uint64_t total = (uint64_t)rows * t.k_storage;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = decode_value(t, expert, row0 + (uint32_t)(i / t.k_storage), (uint32_t)(i % t.k_storage));
}
static DevTensor as_dev(const QW4ShTensor &s) {
    DevTensor t;
    t.data = s.data; t.type = s.type; t.k_storage = s.k_storage; t.k_logical = s.k_logical;
    t.n_out = s.n_out; t.n_experts = s.n_experts; t.row_bytes = s.row_bytes; t.expert_bytes = s.expert_bytes;
    return t;
}
extern "C" int qw4sh_decode_rows(const QW4ShTensor *t, size_t expert, size_t row0, size_t rows, float *out, void *stream) {
    if (!rows) return 0;
    decode_rows_kernel<<<592, 256, 0, (cudaStream_t)stream>>>(as_dev(*t), (uint32_t)expert, (uint32_t)row0, (uint32_t)rows, out);
    LAUNCHED("decode_rows_kernel");
    return 0;
}

// ------------------------------------------------------------------------------------
// Router logits.
// Exact: one thread per (token, expert) walks k = 0..K-1 with separately rounded product and
// sum, the reference's order (src/qwen4_packed.c:164-173), so logits carry the CPU path's
// bits.  The weight tile goes through shared memory so that global reads stay coalesced.
// Row `experts` of the grid is the shared expert's gate (a [1, K] F32 tensor).
// ------------------------------------------------------------------------------------
template <int TT>
__global__ void __launch_bounds__(32 * TT) router_exact_kernel(DevTensor router, DevTensor srouter, const float *__restrict__ x,
                                                               uint32_t tokens, float *__restrict__ logits,
                                                               float *__restrict__ shared_logit, uint32_t *status) {
    constexpr int KC = 128;
    __shared__ float ws[32][KC + 1];
    __shared__ float xs[TT][KC];
    const uint32_t experts = router.n_out, k_total = router.k_logical;
    const uint32_t e = blockIdx.x * 32 + threadIdx.x, t = blockIdx.y * TT + threadIdx.y;
    const uint32_t tid = threadIdx.y * 32 + threadIdx.x, nthreads = 32 * TT;
    float sum = 0.0f;
    for (uint32_t k0 = 0; k0 < k_total; k0 += KC) {
        const uint32_t kc = min((uint32_t)KC, k_total - k0);
        for (uint32_t i = tid; i < 32 * KC; i += nthreads) {
            const uint32_t row = i / KC, col = i % KC, ge = blockIdx.x * 32 + row;
            float v = 0.0f;
            if (col < kc && ge <= experts) {
                const float *src = ge < experts ? (const float *)(router.data + (uint64_t)ge * router.row_bytes)
                                                : (const float *)srouter.data;
                v = src[k0 + col];
            }
            ws[row][col] = v;
        }
        for (uint32_t i = tid; i < TT * KC; i += nthreads) {
            const uint32_t row = i / KC, col = i % KC, gt = blockIdx.y * TT + row;
            xs[row][col] = (col < kc && gt < tokens) ? x[(uint64_t)gt * k_total + k0 + col] : 0.0f;
        }
        __syncthreads();
        if (kc == KC) {
#pragma unroll 16
            for (int kk = 0; kk < KC; kk++) sum = __fadd_rn(sum, __fmul_rn(ws[threadIdx.x][kk], xs[threadIdx.y][kk]));
        } else {
            for (uint32_t kk = 0; kk < kc; kk++) sum = __fadd_rn(sum, __fmul_rn(ws[threadIdx.x][kk], xs[threadIdx.y][kk]));
        }
        __syncthreads();
    }
    if (t < tokens && e <= experts) {
        if (!finite_f32(sum)) atomicOr(status, QW4SH_ERR_NONFINITE);
        if (e < experts) logits[(uint64_t)t * experts + e] = sum;
        else shared_logit[t] = sum;
    }
}

// Exact, mid-sized batches: 16 router rows x 16 tokens per CTA of four warps (one per scheduler), every thread two
// serial chains (one row x two tokens), so that three 128-bit shared-memory reads feed eight chain steps.  Measured
// here: with one chain per thread (256 threads) the kernel is bound by shared-memory bandwidth, with four chains in
// a lone warp per SM by that warp's issue rate (a warp issues at most every other cycle); this is the middle.
// Both tiles go through a four-stage cp.async ring in chunks of 128 columns (three chunks are in flight ahead of
// the adds: more than a DRAM round trip); row pitch 132 floats keeps the reads free of bank conflicts.
constexpr int RC_ROWS = 16, RC_TOK = 16, RC_K = 128, RC_PITCH = 132, RC_STAGES = 4, RC_THREADS = 128;
constexpr size_t RC_SMEM = (size_t)RC_STAGES * (RC_ROWS + RC_TOK) * RC_PITCH * sizeof(float);
__device__ __forceinline__ void rc_copy16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__global__ void __launch_bounds__(RC_THREADS) router_chain_kernel(DevTensor router, DevTensor srouter, const float *__restrict__ x, uint32_t tokens,
                                                                  float *__restrict__ logits, float *__restrict__ shared_logit, uint32_t *status) {
    extern __shared__ __align__(16) uint8_t rc_smem[];
    float (*tile)[RC_ROWS + RC_TOK][RC_PITCH] = reinterpret_cast<float (*)[RC_ROWS + RC_TOK][RC_PITCH]>(rc_smem);   // rows 0-15 router rows, 16-31 tokens
    const uint32_t experts = router.n_out, K = router.k_logical, tid = threadIdx.x;
    const uint32_t e0 = blockIdx.x * RC_ROWS, t0 = blockIdx.y * RC_TOK;
    const uint32_t chunks = K / RC_K;
    // loader role: thread t copies the 16-byte piece t % 32 of rows t / 32, t / 32 + 4, ... (32 pieces = 128 columns)
    const uint32_t piece = (tid & 31u) * 4, lrow = tid >> 5;
    const float *srcs[(RC_ROWS + RC_TOK) / 4];
#pragma unroll
    for (int j = 0; j < (RC_ROWS + RC_TOK) / 4; j++) {
        const uint32_t r = lrow + 4 * j;
        if (r < RC_ROWS) {
            const uint32_t e = e0 + r;
            srcs[j] = (e < experts ? (const float *)(router.data + (uint64_t)e * router.row_bytes) : (const float *)srouter.data) + piece;
        } else srcs[j] = x + (uint64_t)min(t0 + r - RC_ROWS, tokens - 1) * K + piece;
    }
    auto load = [&](uint32_t c) {
        if (c < chunks) {
#pragma unroll
            for (int j = 0; j < (RC_ROWS + RC_TOK) / 4; j++) rc_copy16(&tile[c % RC_STAGES][lrow + 4 * j][piece], srcs[j] + c * RC_K);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (uint32_t c = 0; c + 1 < RC_STAGES; c++) load(c);
    const uint32_t er = tid >> 3, tc = tid & 7u;                                 // worker role: row er x tokens tc, tc + 8
    float s0 = 0.0f, s1 = 0.0f;
    for (uint32_t c = 0; c < chunks; c++) {
        load(c + RC_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(RC_STAGES - 1) : "memory");
        __syncthreads();
        const float4 *w4 = reinterpret_cast<const float4 *>(tile[c % RC_STAGES][er]);
        const float4 *x0 = reinterpret_cast<const float4 *>(tile[c % RC_STAGES][RC_ROWS + tc]), *x1 = reinterpret_cast<const float4 *>(tile[c % RC_STAGES][RC_ROWS + tc + 8]);
#pragma unroll 8
        for (int i = 0; i < RC_K / 4; i++) {
            const float4 a = w4[i], u = x0[i], v = x1[i];
            const float p0 = __fmul_rn(a.x, u.x), p1 = __fmul_rn(a.x, v.x), p2 = __fmul_rn(a.y, u.y), p3 = __fmul_rn(a.y, v.y);
            const float p4 = __fmul_rn(a.z, u.z), p5 = __fmul_rn(a.z, v.z), p6 = __fmul_rn(a.w, u.w), p7 = __fmul_rn(a.w, v.w);
            s0 = __fadd_rn(s0, p0); s1 = __fadd_rn(s1, p1); s0 = __fadd_rn(s0, p2); s1 = __fadd_rn(s1, p3);
            s0 = __fadd_rn(s0, p4); s1 = __fadd_rn(s1, p5); s0 = __fadd_rn(s0, p6); s1 = __fadd_rn(s1, p7);
        }
        __syncthreads();
    }
    const uint32_t e = e0 + er;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const uint32_t t = t0 + tc + 8 * j;
        const float sum = j ? s1 : s0;
        if (t < tokens && e <= experts) {
            bad |= !finite_f32(sum);
            if (e < experts) logits[(uint64_t)t * experts + e] = sum;
            else shared_logit[t] = sum;
        }
    }
    if (bad) atomicOr(status, QW4SH_ERR_NONFINITE);
}

// Exact, few tokens: one warp per (32 router rows, token).  The serial chain of separately
// rounded multiply-adds (the reference's order) is the critical path: K dependent additions.
// To keep operands ahead of the chain, the 32 rows are staged through shared memory by bulk
// copies (one per lane and chunk of 512 columns, three chunks in flight); rows are padded by
// 16 bytes so that the lanes' 128-bit reads fall in different banks.
__device__ __forceinline__ uint32_t rsm_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
constexpr uint32_t RS_CHUNK = 512, RS_PITCH = RS_CHUNK * 4 + 16, RS_STAGES = 3;
__global__ void __launch_bounds__(32) router_exact_small_kernel(DevTensor router, DevTensor srouter, const float *__restrict__ x,
                                                                float *__restrict__ logits, float *__restrict__ shared_logit,
                                                                uint32_t *status) {
    extern __shared__ __align__(128) uint8_t rs_smem[];       // [STAGES][32][PITCH] | x [K] floats | barriers
    const uint32_t experts = router.n_out, K = router.k_logical, lane = threadIdx.x;
    const uint32_t e = blockIdx.x * 32 + lane, t = blockIdx.y;
    const uint8_t *row = e < experts ? router.data + (uint64_t)e * router.row_bytes : (e == experts ? srouter.data : router.data);
    float *xs = reinterpret_cast<float *>(rs_smem + RS_STAGES * 32 * RS_PITCH);
    uint64_t *bar = reinterpret_cast<uint64_t *>(rs_smem + RS_STAGES * 32 * RS_PITCH + ((K * 4 + 15) & ~15u));
    const uint32_t chunks = (K + RS_CHUNK - 1) / RS_CHUNK;
    if (lane == 0) {
        for (uint32_t s = 0; s < RS_STAGES; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(rsm_u32(&bar[s])), "r"(1u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    auto issue = [&](uint32_t c) {
        const uint32_t s = c % RS_STAGES, bytes = min(RS_CHUNK, K - c * RS_CHUNK) * 4;
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rsm_u32(&bar[s])), "r"(bytes * 32) : "memory");
        __syncwarp();
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(rsm_u32(rs_smem + (s * 32 + lane) * RS_PITCH)), "l"(row + (uint64_t)c * RS_CHUNK * 4), "r"(bytes), "r"(rsm_u32(&bar[s])) : "memory");
    };
    for (uint32_t c = 0; c < RS_STAGES && c < chunks; c++) issue(c);
    for (uint32_t k = lane * 4; k < K; k += 128) *reinterpret_cast<float4 *>(xs + k) = *reinterpret_cast<const float4 *>(x + (uint64_t)t * K + k);
    __syncwarp();
    float sum = 0.0f;
    bool alive = true;
    for (uint32_t c = 0; c < chunks; c++) {
        const uint32_t s = c % RS_STAGES, parity = (c / RS_STAGES) & 1u, cols = min(RS_CHUNK, K - c * RS_CHUNK);
        if (alive) {                                           // bounded wait (~1 s), then give up with an error bit
            const long long start = clock64();
            uint32_t ok = 0;
            while (!ok) {
                asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                             : "=r"(ok) : "r"(rsm_u32(&bar[s])), "r"(parity) : "memory");
                if (!ok && clock64() - start > (1ll << 31)) { atomicOr(status, QW4SH_ERR_STATE); alive = false; break; }
            }
        }
        alive = __all_sync(0xffffffffu, alive);
        if (alive) {
            const float4 *w = reinterpret_cast<const float4 *>(rs_smem + (s * 32 + lane) * RS_PITCH);
            const float4 *xv = reinterpret_cast<const float4 *>(xs + c * RS_CHUNK);
#pragma unroll 8
            for (uint32_t i = 0; i < cols / 4; i++) {
                const float4 a = w[i], b = xv[i];
                sum = __fadd_rn(sum, __fmul_rn(a.x, b.x)); sum = __fadd_rn(sum, __fmul_rn(a.y, b.y));
                sum = __fadd_rn(sum, __fmul_rn(a.z, b.z)); sum = __fadd_rn(sum, __fmul_rn(a.w, b.w));
            }
        }
        __syncwarp();
        if (alive && c + RS_STAGES < chunks) issue(c + RS_STAGES);
    }
    if (e <= experts && alive) {
        if (!finite_f32(sum)) atomicOr(status, QW4SH_ERR_NONFINITE);
        if (e < experts) logits[(uint64_t)t * experts + e] = sum;
        else shared_logit[t] = sum;
    }
}

// Fast: one warp per router row, lanes stride K with 128-bit loads, tree sum.  Up to 8 tokens
// per pass share the weight reads.
__global__ void __launch_bounds__(256) router_fast_kernel(DevTensor router, DevTensor srouter, const float *__restrict__ x,
                                                          uint32_t tokens, float *__restrict__ logits,
                                                          float *__restrict__ shared_logit, uint32_t *status) {
    const uint32_t experts = router.n_out, k_total = router.k_logical;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e = blockIdx.x * 8 + warp;
    if (e > experts) return;
    const float *w = e < experts ? (const float *)(router.data + (uint64_t)e * router.row_bytes) : (const float *)srouter.data;
    for (uint32_t t0 = blockIdx.y * 8; t0 < tokens; t0 += gridDim.y * 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const uint32_t nt = min(8u, tokens - t0);
        if ((k_total & 3u) == 0) {
            for (uint32_t k = lane * 4; k < k_total; k += 128) {
                const float4 wv = *reinterpret_cast<const float4 *>(w + k);
#pragma unroll
                for (int r = 0; r < 8; r++) if ((uint32_t)r < nt) {
                    const float4 xv = *reinterpret_cast<const float4 *>(x + (uint64_t)(t0 + r) * k_total + k);
                    acc[r] = fmaf(wv.x, xv.x, fmaf(wv.y, xv.y, fmaf(wv.z, xv.z, fmaf(wv.w, xv.w, acc[r]))));
                }
            }
        } else {
            for (uint32_t k = lane; k < k_total; k += 32)
#pragma unroll
                for (int r = 0; r < 8; r++) if ((uint32_t)r < nt) acc[r] = fmaf(w[k], x[(uint64_t)(t0 + r) * k_total + k], acc[r]);
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
            float v = acc[r];
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && (uint32_t)r < nt) {
                if (!finite_f32(v)) atomicOr(status, QW4SH_ERR_NONFINITE);
                if (e < experts) logits[(uint64_t)(t0 + r) * experts + e] = v;
                else shared_logit[t0 + r] = v;
            }
        }
    }
}

// Router logits for large batches: a register-tiled FP32 GEMM (64 tokens x 64 router rows per
// CTA, 4 x 4 outputs per thread).  Every output still adds its products in ascending k with a
// separately rounded multiply and add when EXACT (the reference's order and bits,
// src/qwen4_packed.c:164-173); outputs are independent chains, so sixteen of them interleave in
// each thread.  Row `experts` is the shared expert's gate.
// TI x TJ outputs per thread (tokens x router rows): a CTA of 256 threads covers 16 TI tokens x 16 TJ rows.  The kernel
// is bound by shared-memory reads and issue slots (two instructions per multiply-add in the exact mode), so the tile
// per thread stays as large as the batch allows while the grid still covers the SMs.  (Packed mul.rn.f32x2 / add.rn.f32x2
// on token pairs was 15% faster but its sums were not the scalar ones in the last bit, so the exact mode stays scalar.)
template <bool EXACT, int TI, int TJ>
__global__ void __launch_bounds__(256) router_gemm_kernel(DevTensor router, DevTensor srouter, const float *__restrict__ x, uint32_t tokens,
                                                          float *__restrict__ logits, float *__restrict__ shared_logit, uint32_t *status) {
    // columns per stage: the narrower the tile of router rows, the less arithmetic a stage holds, so it covers more
    // columns to keep the global-memory round trip of the next stage hidden (two stages of shared memory, <= 45 KB)
    constexpr int BM = 16 * TI, BN = 16 * TJ, BK = TJ >= 2 ? 32 : 64, PASSES = BK / 16;
    __shared__ __align__(16) float xs[2][BK][BM + 4], ws[2][BK][BN + 4];
    const uint32_t experts = router.n_out, K = router.k_logical;
    const uint32_t tid = threadIdx.x, tx = tid & 15u, ty = tid >> 4;
    const uint32_t t0 = blockIdx.x * BM, e0 = blockIdx.y * BN;
    // loader: thread -> (row tid / 4, float4 tid % 4) of each (up to 64) x 16 piece of a stage
    const uint32_t lr = tid >> 2, lc = (tid & 3u) * 4;
    const uint32_t gt = t0 + lr, ge = e0 + lr;
    const bool load_x = lr < BM, load_w = lr < BN;
    const float *xrow = load_x && gt < tokens ? x + (uint64_t)gt * K : nullptr;
    const float *wrow = !load_w ? nullptr : ge < experts ? (const float *)(router.data + (uint64_t)ge * router.row_bytes)
                                                          : (ge == experts ? (const float *)srouter.data : nullptr);
    float acc[TI][TJ];
#pragma unroll
    for (int i = 0; i < TI; i++)
#pragma unroll
        for (int j = 0; j < TJ; j++) acc[i][j] = 0.0f;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 xa[PASSES], wa[PASSES];
#pragma unroll
    for (int q = 0; q < PASSES; q++) {
        xa[q] = xrow ? *reinterpret_cast<const float4 *>(xrow + 16 * q + lc) : zero;
        wa[q] = wrow ? *reinterpret_cast<const float4 *>(wrow + 16 * q + lc) : zero;
    }
    const uint32_t steps = K / BK;
    for (uint32_t s = 0; s < steps; s++) {
        const uint32_t b = s & 1u;
#pragma unroll
        for (int q = 0; q < PASSES; q++) {
            const uint32_t c = 16 * q + lc;
            if (load_x) { xs[b][c][lr] = xa[q].x; xs[b][c + 1][lr] = xa[q].y; xs[b][c + 2][lr] = xa[q].z; xs[b][c + 3][lr] = xa[q].w; }
            if (load_w) { ws[b][c][lr] = wa[q].x; ws[b][c + 1][lr] = wa[q].y; ws[b][c + 2][lr] = wa[q].z; ws[b][c + 3][lr] = wa[q].w; }
        }
        __syncthreads();
        if (s + 1 < steps) {
#pragma unroll
            for (int q = 0; q < PASSES; q++) {
                xa[q] = xrow ? *reinterpret_cast<const float4 *>(xrow + (s + 1) * BK + 16 * q + lc) : zero;
                wa[q] = wrow ? *reinterpret_cast<const float4 *>(wrow + (s + 1) * BK + 16 * q + lc) : zero;
            }
        }
#pragma unroll 16
        for (int kk = 0; kk < BK; kk++) {
            float av[TI], bv[TJ];
#pragma unroll
            for (int i = 0; i < TI; i++) av[i] = xs[b][kk][ty * TI + i];
#pragma unroll
            for (int j = 0; j < TJ; j++) bv[j] = ws[b][kk][tx * TJ + j];
#pragma unroll
            for (int i = 0; i < TI; i++)
#pragma unroll
                for (int j = 0; j < TJ; j++) acc[i][j] = EXACT ? __fadd_rn(acc[i][j], __fmul_rn(bv[j], av[i])) : fmaf(bv[j], av[i], acc[i][j]);
        }
    }
    bool bad = false;
#pragma unroll
    for (int i = 0; i < TI; i++) {
        const uint32_t t = t0 + ty * TI + i;
        if (t >= tokens) continue;
#pragma unroll
        for (int j = 0; j < TJ; j++) {
            const uint32_t e = e0 + tx * TJ + j;
            if (e > experts) continue;
            bad |= !finite_f32(acc[i][j]);
            if (e < experts) logits[(uint64_t)t * experts + e] = acc[i][j];
            else shared_logit[t] = acc[i][j];
        }
    }
    if (bad) atomicOr(status, QW4SH_ERR_NONFINITE);
}

// ------------------------------------------------------------------------------------
// Route: one warp per token (src/qwen4_moe.c:209-247).  The exp-sum runs serially over
// e = 0..E-1 on one lane, the reference's order, so probabilities and weights carry its bits;
// the k argmax rounds are warp-parallel with ties to the lower id (strict > in ascending e).
// ------------------------------------------------------------------------------------
// One token: warp-wide.  p is this warp's shared-memory row of `experts` floats.
__device__ __forceinline__ void route_token(uint32_t experts, uint32_t k, int norm, const float *__restrict__ z, uint32_t t,
                                            float *p, float *__restrict__ probs, uint32_t *__restrict__ ids,
                                            float *__restrict__ weights, uint32_t *status, uint32_t lane) {
    bool bad = false;
    float maximum = -CUDART_INF_F;
    for (uint32_t e = lane; e < experts; e += 32) {
        const float v = z[e];
        bad |= !finite_f32(v);
        maximum = fmaxf(maximum, v);
    }
    bad = __any_sync(0xffffffffu, bad);
    if (bad) {
        if (lane == 0) { atomicOr(status, QW4SH_ERR_NONFINITE); atomicMin(status + 1, t); }
        return;
    }
    for (int o = 16; o; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
    for (uint32_t e = lane; e < experts; e += 32) p[e] = expf_libm(__fsub_rn(z[e], maximum));
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0) {
        uint32_t e = 0;
        for (; e + 8 <= experts; e += 8) {
            const float a0 = p[e], a1 = p[e + 1], a2 = p[e + 2], a3 = p[e + 3], a4 = p[e + 4], a5 = p[e + 5], a6 = p[e + 6], a7 = p[e + 7];
            sum = __fadd_rn(sum, a0); sum = __fadd_rn(sum, a1); sum = __fadd_rn(sum, a2); sum = __fadd_rn(sum, a3);
            sum = __fadd_rn(sum, a4); sum = __fadd_rn(sum, a5); sum = __fadd_rn(sum, a6); sum = __fadd_rn(sum, a7);
        }
        for (; e < experts; e++) sum = __fadd_rn(sum, p[e]);
    }
    sum = __shfl_sync(0xffffffffu, sum, 0);
    for (uint32_t e = lane; e < experts; e += 32) {
        const float v = __fdiv_rn(p[e], sum);
        p[e] = v;
        probs[(uint64_t)t * experts + e] = v;
    }
    __syncwarp();
    float selected = 0.0f;
    for (uint32_t slot = 0; slot < k; slot++) {
        float best = -1.0f;
        uint32_t best_e = 0xffffffffu;
        for (uint32_t e = lane; e < experts; e += 32) {
            const float v = p[e];
            if (v > best) { best = v; best_e = e; }
        }
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (lane == 0) { ids[(uint64_t)t * k + slot] = best_e; weights[(uint64_t)t * k + slot] = best; }
        if ((best_e & 31u) == lane) p[best_e] = -1.0f;         // probabilities are >= 0: never chosen again
        selected = __fadd_rn(selected, best);
        __syncwarp();
    }
    // Lane 0 stored the raw weights above and is the only reader here.
    if (norm && lane == 0)
        for (uint32_t slot = 0; slot < k; slot++)
            weights[(uint64_t)t * k + slot] = __fdiv_rn(weights[(uint64_t)t * k + slot], selected);
}

__global__ void __launch_bounds__(128) route_kernel(uint32_t experts, uint32_t k, int norm, const float *__restrict__ logits,
                                                    uint64_t pitch, uint32_t tokens, float *__restrict__ probs,
                                                    uint32_t *__restrict__ ids, float *__restrict__ weights, uint32_t *status) {
    extern __shared__ float route_smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    const uint32_t t = blockIdx.x * warps + warp;
    if (t >= tokens) return;
    if (experts <= 512 && k <= 32) route_token_regs<16>(experts, k, norm, logits + (uint64_t)t * pitch, t, probs, ids, weights, status, lane);
    else route_token(experts, k, norm, logits + (uint64_t)t * pitch, t, route_smem + (uint64_t)warp * experts, probs, ids, weights, status, lane);
}

// Few tokens: one CTA of 512 threads per token routes it (thread e owns expert e, experts <=
// 512), and the CTA that finishes last builds the stable per-expert lists and the groups of
// <= 4 rows for all tokens (no CTA waits for another: the last one to arrive is found with an
// atomic counter).  One lone warp per token would be bound by its own instruction latency;
// spreading exp, division and the k arg-max rounds over 16 warps leaves only the exp-sum serial
// (512 dependent additions in expert order, the reference's order).
struct Group4 { uint32_t expert, first, count, pad; };
__global__ void __launch_bounds__(512) route_group_small_kernel(uint32_t experts, uint32_t k, int norm, const float *__restrict__ logits,
                                                                uint32_t tokens, float *__restrict__ probs, uint32_t *__restrict__ ids,
                                                                float *__restrict__ weights, uint32_t *__restrict__ offsets,
                                                                uint32_t *__restrict__ pair_to_row, uint32_t *__restrict__ row_to_pair,
                                                                uint32_t *__restrict__ active, Group4 *__restrict__ groups,
                                                                uint32_t *__restrict__ n_groups, uint32_t *status) {
    __shared__ __align__(16) float p[512];
    __shared__ float wred[16];
    __shared__ float s_sum;
    __shared__ uint32_t s_bad, s_last, wsum[16];
    extern __shared__ uint32_t sids[];                         // [tokens * k] for the dispatch step
    const uint32_t t = blockIdx.x, e = threadIdx.x, lane = e & 31u, warp = e >> 5;
    if (e == 0) s_bad = 0;
    __syncthreads();
    float z = e < experts ? logits[(uint64_t)t * experts + e] : -CUDART_INF_F;
    if (e < experts && !finite_f32(z)) s_bad = 1;
    float m = z;
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) wred[warp] = m;
    __syncthreads();
    const bool bad = s_bad != 0;
    if (bad && e == 0) { atomicOr(status, QW4SH_ERR_NONFINITE); atomicMin(status + 1, t); }
    float value = -1.0f;
    if (!bad) {
        float maximum = wred[0];
        for (int w = 1; w < 16; w++) maximum = fmaxf(maximum, wred[w]);
        p[e] = e < experts ? expf_libm(__fsub_rn(z, maximum)) : 0.0f;
        __syncthreads();
        if (e == 0) {                                          // the reference's serial sum, e = 0, 1, 2, ...
            float sum = 0.0f;
            uint32_t i = 0;
            for (; i + 16 <= experts; i += 16) {
                const float4 a = *reinterpret_cast<const float4 *>(p + i), b = *reinterpret_cast<const float4 *>(p + i + 4);
                const float4 c = *reinterpret_cast<const float4 *>(p + i + 8), d = *reinterpret_cast<const float4 *>(p + i + 12);
                sum = __fadd_rn(sum, a.x); sum = __fadd_rn(sum, a.y); sum = __fadd_rn(sum, a.z); sum = __fadd_rn(sum, a.w);
                sum = __fadd_rn(sum, b.x); sum = __fadd_rn(sum, b.y); sum = __fadd_rn(sum, b.z); sum = __fadd_rn(sum, b.w);
                sum = __fadd_rn(sum, c.x); sum = __fadd_rn(sum, c.y); sum = __fadd_rn(sum, c.z); sum = __fadd_rn(sum, c.w);
                sum = __fadd_rn(sum, d.x); sum = __fadd_rn(sum, d.y); sum = __fadd_rn(sum, d.z); sum = __fadd_rn(sum, d.w);
            }
            for (; i < experts; i++) sum = __fadd_rn(sum, p[i]);
            s_sum = sum;
        }
        __syncthreads();
        if (e < experts) { value = __fdiv_rn(p[e], s_sum); probs[(uint64_t)t * experts + e] = value; }
        // Selection by one warp over the row in shared memory: lane L owns experts L, L + 32, ... and keeps the best
        // three of them in registers (keys: float bits + 1, a chosen entry becomes -1 = key 0), so a slot costs two
        // warp reductions; a lane rescans its experts only when it wins a third time after its last scan.  Ties go
        // to the lower id, the sum of the chosen probabilities runs in slot order (the reference's order).
        __syncthreads();                                       // every thread has read its exp value out of p
        p[e] = e < experts ? value : -1.0f;
        __syncthreads();
        if (warp == 0) {
            uint32_t b1, e1, b2, e2, b3, e3;
            auto scan3 = [&]() {
                b1 = 0; e1 = 0xffffffffu; b2 = 0; e2 = 0xffffffffu; b3 = 0; e3 = 0xffffffffu;
#pragma unroll 4
                for (uint32_t i = lane; i < experts; i += 32) {            // ascending ids: the lowest wins among equals
                    const float v = p[i];
                    const uint32_t key = v < 0.0f ? 0u : __float_as_uint(v) + 1u;
                    if (key > b1) { b3 = b2; e3 = e2; b2 = b1; e2 = e1; b1 = key; e1 = i; }
                    else if (key > b2) { b3 = b2; e3 = e2; b2 = key; e2 = i; }
                    else if (key > b3) { b3 = key; e3 = i; }
                }
            };
            scan3();
            uint32_t spare = 2;
            float selected = 0.0f;
            for (uint32_t slot = 0; slot < k; slot++) {
                const uint32_t top = __reduce_max_sync(0xffffffffu, b1);
                const uint32_t e_win = __reduce_min_sync(0xffffffffu, b1 == top ? e1 : 0xffffffffu);
                const float best = __uint_as_float(top - 1u);
                if (lane == 0) { ids[(uint64_t)t * k + slot] = e_win; sids[slot] = top - 1u; }    // sids: free until the dispatch step
                if ((e_win & 31u) == lane) {
                    p[e_win] = -1.0f;
                    if (spare) { b1 = b2; e1 = e2; b2 = b3; e2 = e3; spare--; }
                    else { scan3(); spare = 2; }
                }
                selected = __fadd_rn(selected, best);
            }
            __syncwarp();
            for (uint32_t slot = lane; slot < k; slot += 32) {
                const float raw = __uint_as_float(sids[slot]);
                weights[(uint64_t)t * k + slot] = norm ? __fdiv_rn(raw, selected) : raw;
            }
        }
    }
    // ---- the CTA that arrives last does the dispatch for all tokens ----
    __threadfence();
    __syncthreads();
    if (e == 0) s_last = atomicAdd(n_groups + 2, 1u) == tokens - 1 ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    if (e == 0) n_groups[2] = 0;                                // ready for the next call
    __threadfence();
    // An expert takes a token at most once, so its list is a 64-bit set of tokens (tokens <= 64): thread q marks
    // pair q, thread e counts its set, and every pair finds its own row with one popcount.
    const uint32_t pairs = tokens * k;
    __shared__ unsigned long long s_tokens[512];
    __shared__ uint32_t s_first[512];
    s_tokens[e] = 0ull;
    __syncthreads();
    for (uint32_t q = e; q < pairs; q += blockDim.x) {
        const uint32_t id = __ldcg(ids + q);
        sids[q] = id;
        if (id < experts) atomicOr(&s_tokens[id], 1ull << (q / k));
    }
    __syncthreads();
    const unsigned long long my_tokens = e < experts ? s_tokens[e] : 0ull;
    const uint32_t count = __popcll(my_tokens);
    // packed: bits 0-11 rows, 12-21 groups of four, 22-31 non-empty flag
    const uint32_t packed = count | (((count + 3) >> 2) << 12) | ((count ? 1u : 0u) << 22);
    uint32_t scan = packed;
    for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(0xffffffffu, scan, o); if (lane >= (uint32_t)o) scan += v; }
    if (lane == 31) wsum[warp] = scan;
    __syncthreads();
    if (warp == 0) {
        uint32_t v = lane < 16 ? wsum[lane] : 0, sc = v;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, sc, o); if (lane >= (uint32_t)o) sc += u; }
        if (lane < 16) wsum[lane] = sc - v;
    }
    __syncthreads();
    const uint32_t exclusive = scan - packed + wsum[warp];
    const uint32_t first = exclusive & 0xfffu, gfirst = (exclusive >> 12) & 0x3ffu, arank = exclusive >> 22;
    if (e < experts) {
        offsets[e] = first;
        if (count) {
            active[1 + arank] = e;
            for (uint32_t j = 0; j < (count + 3) >> 2; j++) groups[gfirst + j] = Group4{e, first + 4 * j, min(4u, count - 4 * j), 0};
        }
    }
    // placement by pair: a pair's row is its expert's first row plus the number of lower tokens in the expert's set
    s_first[e] = first;
    __syncthreads();
    for (uint32_t q = e; q < pairs; q += blockDim.x) {
        const uint32_t id = sids[q];
        if (id < experts) {
            const uint32_t row = s_first[id] + __popcll(s_tokens[id] & ((1ull << (q / k)) - 1ull));
            pair_to_row[q] = row; row_to_pair[row] = q;
        }
    }
    if (e == blockDim.x - 1) {                                   // inclusive total sits in the last thread
        const uint32_t total = exclusive + packed;
        offsets[experts] = total & 0xfffu; n_groups[0] = (total >> 12) & 0x3ffu; active[0] = total >> 22;
    }
    for (uint32_t j = e; j < (tokens + 3) / 4; j += blockDim.x)   // the shared expert's groups: rows four at a time
        groups[pairs + j] = Group4{0, 4 * j, min(4u, tokens - 4 * j), 0};
    if (e == 0) n_groups[1] = (tokens + 3) / 4;
}

// ------------------------------------------------------------------------------------
// Dispatch: stable counting sort of pair = t*k + slot by expert (src/qwen4_moe.c:285-301),
// one CTA.  Order inside an expert is by ascending pair, so the lists equal the CPU path's.
// Thread e owns expert e: it counts, then walks the pairs in order and places its own.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) group_kernel(uint32_t experts, uint32_t pairs, const uint32_t *__restrict__ ids,
                                                     uint32_t *__restrict__ offsets, uint32_t *__restrict__ pair_to_row,
                                                     uint32_t *__restrict__ row_to_pair, uint32_t *__restrict__ active, uint32_t *status) {
    extern __shared__ uint32_t group_smem[];                   // counts[experts + 1]
    uint32_t *counts = group_smem;
    for (uint32_t e = threadIdx.x; e <= experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    bool bounds = false;
    for (uint32_t p = threadIdx.x; p < pairs; p += blockDim.x) {
        const uint32_t e = ids[p];
        if (e < experts) atomicAdd(&counts[e], 1u); else if (e != 0xffffffffu) bounds = true;   // 0xffffffff: no expert, skipped
    }
    if (bounds) atomicOr(status, QW4SH_ERR_BOUNDS);
    __syncthreads();
    if (threadIdx.x == 0) {                                    // exclusive prefix; E is small
        uint32_t running = 0, n_active = 0;
        for (uint32_t e = 0; e < experts; e++) {
            const uint32_t c = counts[e];
            counts[e] = running;
            offsets[e] = running;
            if (c) active[1 + n_active++] = e;
            running += c;
        }
        counts[experts] = running;
        offsets[experts] = running;
        active[0] = n_active;
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) {
        uint32_t cursor = counts[e];
        const uint32_t end = counts[e + 1];
        for (uint32_t p = 0; p < pairs && cursor < end; p++)
            if (ids[p] == e) { pair_to_row[p] = cursor; row_to_pair[cursor] = p; cursor++; }
    }
}

// Dispatch of plain rows (one expert id per row, any id any number of times; 0xffffffff: no expert), as the
// expert-parallel owner sees them: stable counting sort in one CTA.  Counts by shared-memory atomics, a block scan
// over the experts, then placement in row order: within a warp a row's rank among equal ids comes from
// __match_any_sync, and the warps of a round of 1024 rows take turns at the per-expert cursors, so the order inside
// an expert is by ascending row.  experts <= 1024.
__global__ void __launch_bounds__(1024) group_rows_kernel(uint32_t experts, uint32_t rows, const uint32_t *__restrict__ ids,
                                                          uint32_t *__restrict__ offsets, uint32_t *__restrict__ pair_to_row,
                                                          uint32_t *__restrict__ row_to_pair, uint32_t *__restrict__ active, uint32_t *status) {
    __shared__ uint32_t cursor[1024];
    __shared__ uint32_t wsum[32];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    cursor[tid] = 0;
    __syncthreads();
    bool bounds = false;
    for (uint32_t r = tid; r < rows; r += 1024) {
        const uint32_t e = ids[r];
        if (e < experts) atomicAdd(&cursor[e], 1u); else if (e != 0xffffffffu) bounds = true;
    }
    if (bounds) atomicOr(status, QW4SH_ERR_BOUNDS);
    __syncthreads();
    // packed scan: rows in bits 0-19, non-empty experts from bit 20
    const uint32_t count = tid < experts ? cursor[tid] : 0, packed = count | ((count ? 1u : 0u) << 20);
    uint32_t scan = packed;
    for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(0xffffffffu, scan, o); if (lane >= (uint32_t)o) scan += v; }
    if (lane == 31) wsum[warp] = scan;
    __syncthreads();
    if (warp == 0) {
        const uint32_t v = wsum[lane];
        uint32_t sc = v;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, sc, o); if (lane >= (uint32_t)o) sc += u; }
        wsum[lane] = sc - v;
    }
    __syncthreads();
    const uint32_t exclusive = wsum[warp] + scan - packed, first = exclusive & 0xfffffu;
    if (tid < experts) {
        offsets[tid] = first;
        if (count) active[1 + (exclusive >> 20)] = tid;
    }
    if (tid == 1023) { offsets[experts] = (exclusive + packed) & 0xfffffu; active[0] = (exclusive + packed) >> 20; }
    __syncthreads();
    cursor[tid] = first;
    __syncthreads();
    for (uint32_t r0 = 0; r0 < rows; r0 += 1024) {
        const uint32_t r = r0 + tid;
        const uint32_t e = r < rows ? ids[r] : 0xffffffffu;
        const bool ok = e < experts;
        const uint32_t same = __match_any_sync(0xffffffffu, ok ? e : 0xffffffffu);
        const uint32_t rank = __popc(same & ((1u << lane) - 1u)), leader = __ffs(same) - 1;
        const uint32_t warps = min(32u, (rows - r0 + 31) / 32);
        uint32_t base = 0;
        for (uint32_t w = 0; w < warps; w++) {                     // the warps of this batch in turn: stable across warps
            if (warp == w && ok && rank == 0) { base = cursor[e]; cursor[e] = base + __popc(same); }
            __syncthreads();
        }
        base = __shfl_sync(0xffffffffu, base, leader);
        if (ok) { pair_to_row[r] = base + rank; row_to_pair[base + rank] = r; }
    }
}

// Dispatch for large batches.  A token routes to an expert at most once, so the order of an
// expert's rows (ascending pair) is the order of its tokens: one bit per (expert, token), and a
// pair's rank inside its expert is the number of set bits below its token.  Four small launches:
// mark bits, per-expert word prefixes and counts, exclusive prefix over experts, placement.
__global__ void __launch_bounds__(256) dispatch_mark_kernel(const uint32_t *__restrict__ ids, uint32_t pairs, uint32_t k, uint32_t experts,
                                                            uint32_t words, uint32_t *bitmap, uint32_t *status) {
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pairs) return;
    const uint32_t e = ids[p], t = p / k;
    if (e < experts) atomicOr(&bitmap[(uint64_t)e * words + (t >> 5)], 1u << (t & 31u));
    else if (e != 0xffffffffu) atomicOr(status, QW4SH_ERR_BOUNDS);
}
__global__ void __launch_bounds__(256) dispatch_count_kernel(const uint32_t *__restrict__ bitmap, uint32_t experts, uint32_t words,
                                                             uint32_t *__restrict__ wordprefix, uint32_t *__restrict__ counts) {
    const uint32_t e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (e >= experts) return;
    uint32_t running = 0;
    for (uint32_t w0 = 0; w0 < words; w0 += 32) {
        const uint32_t w = w0 + lane, c = w < words ? __popc(bitmap[(uint64_t)e * words + w]) : 0;
        uint32_t scan = c;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(0xffffffffu, scan, o); if (lane >= (uint32_t)o) scan += v; }
        if (w < words) wordprefix[(uint64_t)e * words + w] = running + scan - c;
        running += __shfl_sync(0xffffffffu, scan, 31);
    }
    if (lane == 0) counts[e] = running;
}
__global__ void __launch_bounds__(1024) dispatch_offsets_kernel(const uint32_t *__restrict__ counts, uint32_t experts, uint32_t *__restrict__ offsets,
                                                                uint32_t *__restrict__ active) {
    __shared__ uint32_t wsum[32], wact[32];
    __shared__ uint32_t carry[2];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid == 0) { carry[0] = 0; carry[1] = 0; }
    __syncthreads();
    for (uint32_t e0 = 0; e0 < experts; e0 += 1024) {
        const uint32_t e = e0 + tid, c = e < experts ? counts[e] : 0, f = c ? 1u : 0u;
        uint32_t scan = c, ascan = f;
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, scan, o), u = __shfl_up_sync(0xffffffffu, ascan, o);
            if (lane >= (uint32_t)o) { scan += v; ascan += u; }
        }
        if (lane == 31) { wsum[warp] = scan; wact[warp] = ascan; }
        __syncthreads();
        if (warp == 0) {
            const uint32_t v = wsum[lane], u = wact[lane];
            uint32_t sv = v, su = u;
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t a = __shfl_up_sync(0xffffffffu, sv, o), b = __shfl_up_sync(0xffffffffu, su, o);
                if (lane >= (uint32_t)o) { sv += a; su += b; }
            }
            wsum[lane] = sv - v; wact[lane] = su - u;
        }
        __syncthreads();
        const uint32_t first = carry[0] + wsum[warp] + scan - c, rank = carry[1] + wact[warp] + ascan - f;
        if (e < experts) { offsets[e] = first; if (c) active[1 + rank] = e; }
        __syncthreads();
        if (tid == 1023) { carry[0] = first + c; carry[1] = rank + f; }
        __syncthreads();
    }
    if (tid == 0) { offsets[experts] = carry[0]; active[0] = carry[1]; }
}
__global__ void __launch_bounds__(256) dispatch_place_kernel(const uint32_t *__restrict__ ids, uint32_t pairs, uint32_t k, uint32_t experts,
                                                             uint32_t words, const uint32_t *__restrict__ bitmap,
                                                             const uint32_t *__restrict__ wordprefix, const uint32_t *__restrict__ offsets,
                                                             uint32_t *__restrict__ pair_to_row, uint32_t *__restrict__ row_to_pair) {
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pairs) return;
    const uint32_t e = ids[p], t = p / k;
    if (e >= experts) return;
    const uint64_t at = (uint64_t)e * words + (t >> 5);
    const uint32_t row = offsets[e] + wordprefix[at] + __popc(bitmap[at] & ((1u << (t & 31u)) - 1u));
    pair_to_row[p] = row;
    row_to_pair[row] = p;
}
// scratch: 2 * experts * ceil(tokens / 32) + experts words.
extern "C" int qw4sh_group_large(uint32_t experts, uint32_t k, size_t tokens, const uint32_t *ids, uint32_t *offsets, uint32_t *pair_to_row,
                                 uint32_t *row_to_pair, uint32_t *active, uint32_t *scratch, uint32_t *status, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    const uint32_t words = (uint32_t)((tokens + 31) / 32), pairs = (uint32_t)(tokens * k);
    uint32_t *bitmap = scratch, *wordprefix = scratch + (size_t)experts * words, *counts = wordprefix + (size_t)experts * words;
    CU(cudaMemsetAsync(bitmap, 0, (size_t)experts * words * 4, stream));
    dispatch_mark_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(ids, pairs, k, experts, words, bitmap, status);
    LAUNCHED("dispatch_mark_kernel");
    dispatch_count_kernel<<<(experts + 7) / 8, 256, 0, stream>>>(bitmap, experts, words, wordprefix, counts);
    LAUNCHED("dispatch_count_kernel");
    dispatch_offsets_kernel<<<1, 1024, 0, stream>>>(counts, experts, offsets, active);
    LAUNCHED("dispatch_offsets_kernel");
    dispatch_place_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(ids, pairs, k, experts, words, bitmap, wordprefix, offsets, pair_to_row, row_to_pair);
    LAUNCHED("dispatch_place_kernel");
    return 0;
}

// ------------------------------------------------------------------------------------
// Expert products.  Weights are read as 32-weight units (one unit per lane per step):
//   Q4_K     16 B of nibbles: 16 low-nibble weights at col0.. and 16 high-nibble at col0+32..
//   Q2_K      8 B of 2-bit codes: 4 runs of 8 weights, 32 columns apart
//   IQ2_XXS   8 B group: 4 codebook vectors of 8 weights, 32 contiguous columns
// decode_unit writes the 32 decoded weights and the column of each run of 8.
// Activations sit in shared memory with 4 floats of padding after every 32 (index
// k + 4*(k/32)) so that 128-bit reads by consecutive lanes fall in distinct banks.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t xs_index(uint32_t k) { return k + ((k >> 5) << 2); }

template <uint32_t TYPE> struct Unit;

template <> struct Unit<T_Q4_K> {
    __device__ static __forceinline__ void decode(const uint8_t *mat, uint32_t rows, uint32_t nb, uint32_t row, uint32_t unit,
                                                  const uint16_t *, float (&w)[32], uint32_t (&col)[4]) {
        (void)rows;
        const uint32_t b = unit >> 3, i = unit & 7u, cc = i >> 1, h = i & 1u;
        const uint8_t *blk = mat + ((uint64_t)row * nb + b) * 144u;
        const uint4 head = *reinterpret_cast<const uint4 *>(blk);
        const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + i * 16);
        const float d = __half2float(__ushort_as_half((uint16_t)(head.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((uint16_t)(head.x >> 16)));
        const uint8_t sc[12] = {(uint8_t)head.y, (uint8_t)(head.y >> 8), (uint8_t)(head.y >> 16), (uint8_t)(head.y >> 24),
                                (uint8_t)head.z, (uint8_t)(head.z >> 8), (uint8_t)(head.z >> 16), (uint8_t)(head.z >> 24),
                                (uint8_t)head.w, (uint8_t)(head.w >> 8), (uint8_t)(head.w >> 16), (uint8_t)(head.w >> 24)};
        uint32_t s0, m0, s1, m1;
        q4k_scale_min(sc, 2 * cc, s0, m0);
        q4k_scale_min(sc, 2 * cc + 1, s1, m1);
        const float dl0 = d * (float)s0, ml0 = dmin * (float)m0, dl1 = d * (float)s1, ml1 = dmin * (float)m1;
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const uint32_t byte = (words[j >> 2] >> ((j & 3) * 8)) & 0xffu;
            w[j] = fmaf(dl0, (float)(byte & 15u), -ml0);
            w[16 + j] = fmaf(dl1, (float)(byte >> 4), -ml1);
        }
        const uint32_t col0 = b * 256 + cc * 64 + h * 16;
        col[0] = col0; col[1] = col0 + 8; col[2] = col0 + 32; col[3] = col0 + 40;
    }
};

template <> struct Unit<T_Q2_K> {
    __device__ static __forceinline__ void decode(const uint8_t *mat, uint32_t rows, uint32_t nb, uint32_t row, uint32_t unit,
                                                  const uint16_t *, float (&w)[32], uint32_t (&col)[4]) {
        const uint32_t b = unit >> 3, i = unit & 7u, hh = i >> 2, ii = i & 3u;
        const uint64_t blocks = (uint64_t)rows * nb, block = (uint64_t)row * nb + b;
        const uint2 codes = *reinterpret_cast<const uint2 *>(mat + block * 64u + hh * 32 + ii * 8);
        const uint8_t *scales = mat + blocks * 64u + block * 16u;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(mat + blocks * 80u + block * 4u);
        const float d = __half2float(__ushort_as_half((uint16_t)(dd & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((uint16_t)(dd >> 16)));
        const uint32_t words[2] = {codes.x, codes.y};
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t column = hh * 128 + q * 32 + ii * 8;       // within the block
            const uint32_t s = scales[column >> 4];
            const float dl = d * (float)(s & 15u), ml = dmin * (float)(s >> 4);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t byte = (words[j >> 2] >> ((j & 3) * 8)) & 0xffu;
                w[q * 8 + j] = fmaf(dl, (float)((byte >> (2 * q)) & 3u), -ml);
            }
            col[q] = b * 256 + column;
        }
    }
};

template <> struct Unit<T_IQ2_XXS> {
    __device__ static __forceinline__ void decode(const uint8_t *mat, uint32_t rows, uint32_t nb, uint32_t row, uint32_t unit,
                                                  const uint16_t *levels_lut, float (&w)[32], uint32_t (&col)[4]) {
        const uint32_t b = unit >> 3, g = unit & 7u;
        const uint64_t blocks = (uint64_t)rows * nb, block = (uint64_t)row * nb + b;
        const uint2 group = *reinterpret_cast<const uint2 *>(mat + ((uint64_t)row * nb * 8u + ((b * 8u + g) ^ iq2_swizzle(row, nb))) * 8u);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(mat + blocks * 64u + block * 2u)));
        const float scale = d * (float)(2u * (group.y >> 28) + 1u) * 0.125f;
#pragma unroll
        for (int slot = 0; slot < 4; slot++) {
            const uint32_t levels = levels_lut[(group.x >> (8 * slot)) & 0xffu];
            const uint32_t signs = iq2_signs8((group.y >> (7 * slot)) & 127u);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t level = (levels >> (2 * j)) & 3u;
                const float value = scale * (float)iq2_magnitude(level);
                w[slot * 8 + j] = __uint_as_float(__float_as_uint(value) ^ (((signs >> j) & 1u) << 31));
            }
            col[slot] = b * 256 + g * 32 + slot * 8;
        }
    }
};

// acc[r] += sum over the unit's 32 weights of w * x_r, x rows in padded shared memory.
template <int NR>
__device__ __forceinline__ void unit_fma(const float (&w)[32], const uint32_t (&col)[4], const float *xs, uint32_t x_pitch,
                                         uint32_t k_logical, float (&acc)[NR]) {
#pragma unroll
    for (int run = 0; run < 4; run++) {
        if (col[run] >= k_logical) continue;                   // stored padding columns are never read
        const uint32_t at = xs_index(col[run]);
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const float4 a = *reinterpret_cast<const float4 *>(xs + r * x_pitch + at);
            const float4 b = *reinterpret_cast<const float4 *>(xs + r * x_pitch + at + 4);
            float s = acc[r];
            s = fmaf(w[run * 8 + 0], a.x, s); s = fmaf(w[run * 8 + 1], a.y, s);
            s = fmaf(w[run * 8 + 2], a.z, s); s = fmaf(w[run * 8 + 3], a.w, s);
            s = fmaf(w[run * 8 + 4], b.x, s); s = fmaf(w[run * 8 + 5], b.y, s);
            s = fmaf(w[run * 8 + 6], b.z, s); s = fmaf(w[run * 8 + 7], b.w, s);
            acc[r] = s;
        }
    }
}

// Any-format fallback: the unit is 32 consecutive columns decoded one by one.
template <> struct Unit<0xffffffffu> {};

constexpr int GU_ROWS = 4;            // token rows per pass in gate_up
constexpr int GU_WARPS = 8;
constexpr int GU_TILE = 16;           // output rows per CTA

// act[pair, n] = silu(gate_e[n] . x) * (up_e[n] . x) for every pair routed to expert e.
// grid = (ceil(inter / GU_TILE), groups); group g of the grid is expert active[1 + g].
// row_to_pair == nullptr means one group holding rows 0..tokens-1 of x (the shared expert).
template <uint32_t TYPE>
__global__ void __launch_bounds__(GU_WARPS * 32) gate_up_kernel(DevTensor gate, DevTensor up, const float *__restrict__ x,
                                                                uint32_t hidden, const uint32_t *__restrict__ offsets,
                                                                const uint32_t *__restrict__ row_to_pair,
                                                                const uint32_t *__restrict__ active, uint32_t k_div, uint32_t tokens,
                                                                float *__restrict__ act, uint32_t *status) {
    extern __shared__ __align__(16) float gu_smem[];
    __shared__ uint16_t levels_lut[256];
    const uint32_t inter = gate.n_out, nb = gate.k_storage >> 8, units = gate.k_storage >> 5;
    const uint32_t x_pitch = xs_index(hidden) + 4;
    uint32_t expert = 0, first = 0, count = tokens;
    if (row_to_pair) {
        if (blockIdx.y >= active[0]) return;
        expert = active[1 + blockIdx.y];
        first = offsets[expert];
        count = offsets[expert + 1] - first;
    }
    if (TYPE == T_IQ2_XXS) for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) levels_lut[i] = c_iq2_levels[i];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint8_t *gmat = gate.data + (uint64_t)expert * gate.expert_bytes, *umat = up.data + (uint64_t)expert * up.expert_bytes;
    for (uint32_t r0 = 0; r0 < count; r0 += GU_ROWS) {
        const uint32_t nr = min((uint32_t)GU_ROWS, count - r0);
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < GU_ROWS * (hidden >> 2); i += blockDim.x) {
            const uint32_t r = i / (hidden >> 2), c4 = i % (hidden >> 2);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < nr) {
                const uint32_t src_row = row_to_pair ? row_to_pair[first + r0 + r] / k_div : r0 + r;
                v = *reinterpret_cast<const float4 *>(x + (uint64_t)src_row * hidden + c4 * 4);
            }
            *reinterpret_cast<float4 *>(gu_smem + r * x_pitch + xs_index(c4 * 4)) = v;
        }
        __syncthreads();
        for (uint32_t j = warp; j < GU_TILE; j += GU_WARPS) {
            const uint32_t n = blockIdx.x * GU_TILE + j;
            if (n >= inter) break;
            float ag[GU_ROWS] = {0, 0, 0, 0}, au[GU_ROWS] = {0, 0, 0, 0};
            for (uint32_t u = lane; u < units; u += 32) {
                float w[32];
                uint32_t col[4];
                Unit<TYPE>::decode(gmat, inter, nb, n, u, levels_lut, w, col);
                unit_fma<GU_ROWS>(w, col, gu_smem, x_pitch, gate.k_logical, ag);
                Unit<TYPE>::decode(umat, inter, nb, n, u, levels_lut, w, col);
                unit_fma<GU_ROWS>(w, col, gu_smem, x_pitch, gate.k_logical, au);
            }
#pragma unroll
            for (int r = 0; r < GU_ROWS; r++) {
                float g = ag[r], v = au[r];
                for (int o = 16; o; o >>= 1) { g += __shfl_xor_sync(0xffffffffu, g, o); v += __shfl_xor_sync(0xffffffffu, v, o); }
                if (lane == 0 && (uint32_t)r < nr) {
                    const float a = __fmul_rn(__fmul_rn(g, sigmoid_libm(g)), v);
                    if (!finite_f32(a)) atomicOr(status, QW4SH_ERR_NONFINITE);
                    const uint32_t dst = row_to_pair ? row_to_pair[first + r0 + r] : r0 + r;
                    act[(uint64_t)dst * inter + n] = a;
                }
            }
        }
    }
}

// Any-format version (one lane per column, exact decode_value): covers F32/F16/BF16/Q8_0/
// MXFP4 tensors and shapes whose K is not a multiple of 256.
__global__ void __launch_bounds__(256) gate_up_generic_kernel(DevTensor gate, DevTensor up, const float *__restrict__ x,
                                                              uint32_t hidden, const uint32_t *__restrict__ offsets,
                                                              const uint32_t *__restrict__ row_to_pair,
                                                              const uint32_t *__restrict__ active, uint32_t k_div, uint32_t tokens,
                                                              float *__restrict__ act, uint32_t *status) {
    const uint32_t inter = gate.n_out;
    uint32_t expert = 0, first = 0, count = tokens;
    if (row_to_pair) {
        if (blockIdx.y >= active[0]) return;
        expert = active[1 + blockIdx.y];
        first = offsets[expert];
        count = offsets[expert + 1] - first;
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    for (uint32_t n = blockIdx.x * 8 + warp; n < inter; n += gridDim.x * 8)
        for (uint32_t r = 0; r < count; r++) {
            const uint32_t pair = row_to_pair ? row_to_pair[first + r] : r;
            const float *xr = x + (uint64_t)(row_to_pair ? pair / k_div : pair) * hidden;
            float g = 0.f, v = 0.f;
            for (uint32_t c = lane; c < gate.k_logical; c += 32) {
                g = fmaf(decode_value(gate, expert, n, c), xr[c], g);
                v = fmaf(decode_value(up, expert, n, c), xr[c], v);
            }
            for (int o = 16; o; o >>= 1) { g += __shfl_xor_sync(0xffffffffu, g, o); v += __shfl_xor_sync(0xffffffffu, v, o); }
            if (lane == 0) {
                const float a = __fmul_rn(__fmul_rn(g, sigmoid_libm(g)), v);
                if (!finite_f32(a)) atomicOr(status, QW4SH_ERR_NONFINITE);
                act[(uint64_t)pair * inter + n] = a;
            }
        }
}

// y[t, c] = sum over slots (in slot order) of weight[t,s] * (down_e[c] . act[t*k+s])
//           + sigmoid(shared_logit[t]) * (shared_down[c] . shared_act[t])
// (src/qwen4_moe.c:362-380).  grid = (ceil(hidden / DR_TILE), tokens).
constexpr int DR_WARPS = 8;
constexpr int DR_TILE = 64;

template <uint32_t TYPE>
__device__ __forceinline__ float row_dot(const DevTensor &t, const uint8_t *mat, uint32_t row, const float *xs,
                                         const uint16_t *levels_lut, uint32_t lane) {
    float acc[1] = {0.f};
    const uint32_t nb = t.k_storage >> 8, units = t.k_storage >> 5;
    for (uint32_t u = lane; u < units; u += 32) {
        float w[32];
        uint32_t col[4];
        Unit<TYPE>::decode(mat, t.n_out, nb, row, u, levels_lut, w, col);
        unit_fma<1>(w, col, xs, 0, t.k_logical, acc);
    }
    float v = acc[0];
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <>
__device__ __forceinline__ float row_dot<0xffffffffu>(const DevTensor &t, const uint8_t *mat, uint32_t row, const float *xs,
                                                       const uint16_t *, uint32_t lane) {
    float v = 0.f;
    const uint32_t expert = (uint32_t)((mat - t.data) / (t.expert_bytes ? t.expert_bytes : 1));
    for (uint32_t c = lane; c < t.k_logical; c += 32) v = fmaf(decode_value(t, expert, row, c), xs[xs_index(c)], v);
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <uint32_t RT, uint32_t ST>
__global__ void __launch_bounds__(DR_WARPS * 32) down_reduce_kernel(DevTensor down, DevTensor sdown, const float *__restrict__ act,
                                                                    const float *__restrict__ shared_act,
                                                                    const uint32_t *__restrict__ ids, const float *__restrict__ weights,
                                                                    const float *__restrict__ shared_logit, uint32_t k,
                                                                    float *__restrict__ y, float *__restrict__ routed, uint32_t *status) {
    extern __shared__ __align__(16) float dr_smem[];
    __shared__ uint16_t levels_lut[256];
    const uint32_t t = blockIdx.y, hidden = down.n_out, inter = down.k_logical, sinter = sdown.k_logical;
    const uint32_t a_pitch = xs_index(inter) + 4;
    float *sa = dr_smem + (uint64_t)k * a_pitch;
    if (RT == T_IQ2_XXS || ST == T_IQ2_XXS) for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) levels_lut[i] = c_iq2_levels[i];
    for (uint32_t i = threadIdx.x; i < k * inter; i += blockDim.x) {
        const uint32_t s = i / inter, c = i % inter;
        dr_smem[s * a_pitch + xs_index(c)] = act[((uint64_t)t * k + s) * inter + c];
    }
    if (shared_act) for (uint32_t i = threadIdx.x; i < sinter; i += blockDim.x) sa[xs_index(i)] = shared_act[(uint64_t)t * sinter + i];
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const float gate = shared_act ? sigmoid_libm(shared_logit[t]) : 0.0f;
    for (uint32_t j = warp; j < DR_TILE; j += DR_WARPS) {
        const uint32_t c = blockIdx.x * DR_TILE + j;
        if (c >= hidden) break;
        float sum = 0.f;
        bool bad = false;
        for (uint32_t s = 0; s < k; s++) {
            const uint32_t e = ids[(uint64_t)t * k + s];
            if (e == 0xffffffffu) continue;                    // no expert for this row (expert-parallel padding)
            if (e >= down.n_experts) { bad = true; continue; }
            const float dot = row_dot<RT>(down, down.data + (uint64_t)e * down.expert_bytes, c, dr_smem + s * a_pitch, levels_lut, lane);
            sum = __fadd_rn(sum, __fmul_rn(weights ? weights[(uint64_t)t * k + s] : 1.0f, dot));
        }
        const float sdot = shared_act ? row_dot<ST>(sdown, sdown.data, c, sa, levels_lut, lane) : 0.0f;
        const float out = __fadd_rn(sum, __fmul_rn(gate, sdot));
        if (lane == 0) {
            if (bad) atomicOr(status, QW4SH_ERR_BOUNDS);
            if (!finite_f32(out) || !finite_f32(sum)) atomicOr(status, QW4SH_ERR_NONFINITE);
            if (routed) routed[(uint64_t)t * hidden + c] = sum;
            y[(uint64_t)t * hidden + c] = out;
        }
    }
}


// ------------------------------------------------------------------------------------
// Launch helpers
// ------------------------------------------------------------------------------------
static const uint32_t GENERIC = 0xffffffffu;
static uint32_t kernel_type(uint32_t type, uint32_t k_storage) {
    return ((type == T_Q4_K || type == T_Q2_K || type == T_IQ2_XXS) && k_storage % 256 == 0) ? type : GENERIC;
}
static size_t xs_floats(size_t k) { return k + ((k >> 5) << 2) + 4; }

template <typename Kernel>
static int allow_smem(Kernel kernel, size_t smem) {
    if (smem > 227u * 1024u) return fail(cudaErrorInvalidValue, "shape needs more shared memory than one CTA has");
    if (smem > 48u * 1024u) CU(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return 0;
}

extern "C" int qw4sh_route(uint32_t experts, uint32_t k, int norm, const float *logits, size_t pitch, size_t tokens,
                           float *probs, uint32_t *ids, float *weights, uint32_t *status, void *stream) {
    if (!tokens) return 0;
    if (ensure_constants()) return -1;
    const size_t per_warp = (size_t)experts * sizeof(float);
    int warps = 4;
    while (warps > 1 && per_warp * warps > 96u * 1024u) warps >>= 1;
    const size_t smem = per_warp * warps;
    if (allow_smem(route_kernel, smem)) return -1;
    const unsigned blocks = (unsigned)((tokens + warps - 1) / warps);
    route_kernel<<<blocks, warps * 32, smem, (cudaStream_t)stream>>>(experts, k, norm, logits, pitch, (uint32_t)tokens, probs, ids, weights, status);
    LAUNCHED("route_kernel");
    return 0;
}

extern "C" int qw4sh_group(uint32_t experts, uint32_t k, size_t tokens, const uint32_t *ids, uint32_t *offsets,
                           uint32_t *pair_to_row, uint32_t *row_to_pair, uint32_t *active, uint32_t *status, void *stream) {
    const size_t smem = ((size_t)experts + 1) * sizeof(uint32_t);
    if (allow_smem(group_kernel, smem)) return -1;
    group_kernel<<<1, 1024, smem, (cudaStream_t)stream>>>(experts, (uint32_t)(tokens * k), ids, offsets, pair_to_row, row_to_pair, active, status);
    LAUNCHED("group_kernel");
    return 0;
}

static int launch_router(const QW4ShLayer *layer, const float *x, size_t tokens, float *logits, float *shared_logit,
                         uint32_t *status, int mode, cudaStream_t stream) {
    const DevTensor router = as_dev(layer->w[0]), srouter = as_dev(layer->w[7]);
    const uint32_t rows = layer->experts + 1;
    if (mode == 0 && tokens > 4 && tokens <= 128 && router.k_logical % RC_K == 0 && ((uintptr_t)x & 15u) == 0 && router.row_bytes % 16 == 0 &&
               ((uintptr_t)router.data & 15u) == 0 && ((uintptr_t)srouter.data & 15u) == 0) {
        if (allow_smem(router_chain_kernel, RC_SMEM)) return -1;
        router_chain_kernel<<<dim3((rows + RC_ROWS - 1) / RC_ROWS, (unsigned)((tokens + RC_TOK - 1) / RC_TOK)), RC_THREADS, RC_SMEM, stream>>>(
            router, srouter, x, (uint32_t)tokens, logits, shared_logit, status);
        LAUNCHED("router_chain_kernel");
    } else if (mode == 0 && tokens <= 16 && router.k_logical % 4 == 0 && router.k_logical <= 4096) {
        const size_t smem = RS_STAGES * 32 * RS_PITCH + (((size_t)router.k_logical * 4 + 15) & ~(size_t)15) + 64;
        if (allow_smem(router_exact_small_kernel, smem)) return -1;
        router_exact_small_kernel<<<dim3((rows + 31) / 32, (unsigned)tokens), 32, smem, stream>>>(router, srouter, x, logits, shared_logit, status);
        LAUNCHED("router_exact_small_kernel");
    } else if (tokens > 16 && router.k_logical % 64 == 0 && ((uintptr_t)x & 15u) == 0 && router.row_bytes % 16 == 0) {
#define ROUTER_GEMM(TI, TJ) do { \
        const dim3 grid((unsigned)((tokens + 16 * TI - 1) / (16 * TI)), (rows + 16 * TJ - 1) / (16 * TJ)); \
        if (mode == 0) router_gemm_kernel<true, TI, TJ><<<grid, 256, 0, stream>>>(router, srouter, x, (uint32_t)tokens, logits, shared_logit, status); \
        else router_gemm_kernel<false, TI, TJ><<<grid, 256, 0, stream>>>(router, srouter, x, (uint32_t)tokens, logits, shared_logit, status); } while (0)
        // four tokens per thread always (one 128-bit read serves four chains); fewer router rows per thread for
        // smaller batches, so that the grid still covers the SMs
        if (tokens >= 768) ROUTER_GEMM(4, 4);
        else if (tokens >= 384) ROUTER_GEMM(4, 2);
        else ROUTER_GEMM(4, 1);
#undef ROUTER_GEMM
        LAUNCHED("router_gemm_kernel");
    } else if (mode == 0) {
        if (tokens <= 1) {
            router_exact_kernel<1><<<dim3((rows + 31) / 32, (unsigned)tokens), dim3(32, 1), 0, stream>>>(router, srouter, x, (uint32_t)tokens, logits, shared_logit, status);
        } else if (tokens <= 4) {
            router_exact_kernel<4><<<dim3((rows + 31) / 32, (unsigned)((tokens + 3) / 4)), dim3(32, 4), 0, stream>>>(router, srouter, x, (uint32_t)tokens, logits, shared_logit, status);
        } else {
            router_exact_kernel<8><<<dim3((rows + 31) / 32, (unsigned)((tokens + 7) / 8)), dim3(32, 8), 0, stream>>>(router, srouter, x, (uint32_t)tokens, logits, shared_logit, status);
        }
        LAUNCHED("router_exact_kernel");
    } else {
        const unsigned ty = (unsigned)((tokens + 7) / 8);
        router_fast_kernel<<<dim3((rows + 7) / 8, ty > 64 ? 64 : ty), 256, 0, stream>>>(router, srouter, x, (uint32_t)tokens, logits, shared_logit, status);
        LAUNCHED("router_fast_kernel");
    }
    return 0;
}

static int launch_gate_up(const DevTensor &gate, const DevTensor &up, const float *x, uint32_t hidden, const uint32_t *offsets,
                          const uint32_t *row_to_pair, const uint32_t *active, uint32_t k_div, uint32_t tokens, uint32_t groups,
                          float *act, uint32_t *status, cudaStream_t stream) {
    uint32_t type = kernel_type(gate.type, gate.k_storage);
    if (up.type != gate.type || hidden % 4) type = GENERIC;
    const size_t smem = (size_t)GU_ROWS * xs_floats(hidden) * sizeof(float);
    const dim3 grid((gate.n_out + GU_TILE - 1) / GU_TILE, groups);
#define GU_CASE(T) case T: if (allow_smem(gate_up_kernel<T>, smem)) return -1; \
    gate_up_kernel<T><<<grid, GU_WARPS * 32, smem, stream>>>(gate, up, x, hidden, offsets, row_to_pair, active, k_div, tokens, act, status); break;
    switch (type) {
        GU_CASE(T_Q4_K) GU_CASE(T_Q2_K) GU_CASE(T_IQ2_XXS)
    default: {
        const unsigned gx = (gate.n_out + 7) / 8;
        gate_up_generic_kernel<<<dim3(gx > 256 ? 256 : gx, groups), 256, 0, stream>>>(gate, up, x, hidden, offsets, row_to_pair, active, k_div, tokens, act, status);
    }
    }
#undef GU_CASE
    LAUNCHED("gate_up_kernel");
    return 0;
}

template <uint32_t RT>
static int launch_down_st(uint32_t st, const DevTensor &down, const DevTensor &sdown, const float *act, const float *shared_act,
                          const uint32_t *ids, const float *weights, const float *shared_logit, uint32_t k, uint32_t tokens,
                          float *y, float *routed, uint32_t *status, cudaStream_t stream) {
    const size_t smem = ((size_t)k * xs_floats(down.k_logical) + xs_floats(sdown.k_logical)) * sizeof(float);
    const dim3 grid((down.n_out + DR_TILE - 1) / DR_TILE, tokens);
#define DR_CASE(S) case S: if (allow_smem(down_reduce_kernel<RT, S>, smem)) return -1; \
    down_reduce_kernel<RT, S><<<grid, DR_WARPS * 32, smem, stream>>>(down, sdown, act, shared_act, ids, weights, shared_logit, k, y, routed, status); break;
    switch (st) {
        DR_CASE(T_Q4_K) DR_CASE(T_Q2_K) DR_CASE(T_IQ2_XXS)
    default:
        if (allow_smem(down_reduce_kernel<RT, GENERIC>, smem)) return -1;
        down_reduce_kernel<RT, GENERIC><<<grid, DR_WARPS * 32, smem, stream>>>(down, sdown, act, shared_act, ids, weights, shared_logit, k, y, routed, status);
    }
#undef DR_CASE
    LAUNCHED("down_reduce_kernel");
    return 0;
}

static int launch_down(const DevTensor &down, const DevTensor &sdown, const float *act, const float *shared_act,
                       const uint32_t *ids, const float *weights, const float *shared_logit, uint32_t k, uint32_t tokens,
                       float *y, float *routed, uint32_t *status, cudaStream_t stream) {
    const uint32_t rt = kernel_type(down.type, down.k_storage), st = kernel_type(sdown.type, sdown.k_storage);
    switch (rt) {
    case T_Q4_K: return launch_down_st<T_Q4_K>(st, down, sdown, act, shared_act, ids, weights, shared_logit, k, tokens, y, routed, status, stream);
    case T_Q2_K: return launch_down_st<T_Q2_K>(st, down, sdown, act, shared_act, ids, weights, shared_logit, k, tokens, y, routed, status, stream);
    case T_IQ2_XXS: return launch_down_st<T_IQ2_XXS>(st, down, sdown, act, shared_act, ids, weights, shared_logit, k, tokens, y, routed, status, stream);
    default: return launch_down_st<GENERIC>(st, down, sdown, act, shared_act, ids, weights, shared_logit, k, tokens, y, routed, status, stream);
    }
}

__global__ void copy_routes_kernel(const uint32_t *ids, const float *weights, uint32_t n, uint32_t *ids_out, float *weights_out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { if (ids_out) ids_out[i] = ids[i]; if (weights_out) weights_out[i] = weights[i]; }
}

// ------------------------------------------------------------------------------------
// Layer forward: direct launches, CUDA-graph replay, or per-stage timing
// ------------------------------------------------------------------------------------
struct GraphCache {
    cudaGraphExec_t exec = nullptr;
    const void *layer = nullptr, *x = nullptr, *y = nullptr, *ids = nullptr, *weights = nullptr;
    size_t tokens = 0;
    int mode = -1, seen = 0;
};
extern "C" void *qw4sh_graph_cache_create(void) { return new GraphCache(); }
extern "C" void qw4sh_graph_cache_destroy(void *cache) {
    GraphCache *c = (GraphCache *)cache;
    if (!c) return;
    if (c->exec) cudaGraphExecDestroy(c->exec);
    delete c;
}
static int g_graph_mode = 0, g_stage_timing = 0;
static unsigned long long g_capture_launches_before = 0;
extern "C" void qw4sh_set_graph_mode(int on) { g_graph_mode = on ? 1 : 0; }
extern "C" int qw4sh_get_graph_mode(void) { return g_graph_mode; }
// Replay cache for a launch sequence the caller enqueues itself (the expert-parallel step).  try: 0 = enqueue
// directly (graphs off, or first sight of this key: the direct run also settles allocations and kernel attributes),
// 1 = an earlier capture was replayed: nothing left to do, 2 = capture has begun: enqueue, then call finish.
extern "C" int qw4sh_graph_try(const QW4ShWork *work, const void *layer, const void *x, const void *y, const void *ids, const void *weights,
                               size_t tokens, int mode) {
    GraphCache *cache = (GraphCache *)work->graph_cache;
    cudaStream_t stream = (cudaStream_t)work->stream;
    if (!g_graph_mode || !cache) return 0;
    const bool same = cache->layer == layer && cache->x == x && cache->y == y && cache->ids == ids && cache->weights == weights &&
                      cache->tokens == tokens && cache->mode == mode;
    if (same && cache->exec) {
        if (cudaGraphLaunch(cache->exec, stream) != cudaSuccess) return fail(cudaGetLastError(), "graph launch") ? -1 : -1;
        __sync_fetch_and_add(&g_launches, (unsigned long long)cache->seen);
        return 1;
    }
    if (!same) {
        if (cache->exec) { cudaGraphExecDestroy(cache->exec); cache->exec = nullptr; }
        cache->layer = layer; cache->x = x; cache->y = y; cache->ids = ids; cache->weights = weights; cache->tokens = tokens; cache->mode = mode;
        return 0;
    }
    g_capture_launches_before = g_launches;
    if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { fail(cudaGetLastError(), "begin capture"); return -1; }
    return 2;
}
extern "C" int qw4sh_graph_finish(const QW4ShWork *work, int enqueue_failed) {
    GraphCache *cache = (GraphCache *)work->graph_cache;
    cudaStream_t stream = (cudaStream_t)work->stream;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream, &graph);
    cache->seen = (int)(g_launches - g_capture_launches_before);
    g_launches = g_capture_launches_before;
    if (enqueue_failed || e != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        cache->layer = nullptr;
        return enqueue_failed ? -1 : fail(e, "graph capture");
    }
    e = cudaGraphInstantiate(&cache->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { cache->exec = nullptr; cache->layer = nullptr; return fail(e, "graph instantiate"); }
    CU(cudaGraphLaunch(cache->exec, stream));
    __sync_fetch_and_add(&g_launches, (unsigned long long)cache->seen);
    return 0;
}

static cudaEvent_t g_stage_event[QW4SH_STAGES + 1] = {nullptr};
static bool g_stage_pending = false;
static double g_stage_ms[QW4SH_STAGES] = {0};
static uint64_t g_stage_forwards = 0;
static int stage_collect() {
    if (!g_stage_pending) return 0;
    CU(cudaEventSynchronize(g_stage_event[QW4SH_STAGES]));
    for (int i = 0; i < QW4SH_STAGES; i++) {
        float ms = 0;
        CU(cudaEventElapsedTime(&ms, g_stage_event[i], g_stage_event[i + 1]));
        g_stage_ms[i] += ms;
    }
    g_stage_forwards++;
    g_stage_pending = false;
    return 0;
}
extern "C" void qw4sh_set_stage_timing(int on) { g_stage_timing = on ? 1 : 0; }
extern "C" int qw4sh_stage_times(double *ms, uint64_t *forwards) {
    if (stage_collect()) return -1;
    for (int i = 0; i < QW4SH_STAGES; i++) { ms[i] = g_stage_ms[i]; g_stage_ms[i] = 0; }
    *forwards = g_stage_forwards;
    g_stage_forwards = 0;
    return 0;
}

extern "C" int qw4sh_mma_supported(const QW4ShTensor *w, int mode);
extern "C" int qw4sh_grouped_mma(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                                 const uint32_t *row_to_pair, uint32_t k_div, const int8_t *digits, const int8_t *negated,
                                 const int *sums, const float *scale, float *out, uint32_t *status, int ctas, void *stream);
extern "C" int qw4sh_quantize_rows(const float *x, uint32_t rows, uint32_t k, int8_t *xq, int8_t *xneg, int *xsum, float *xscale, void *stream);
extern "C" int qw4sh_combine(const float *out, const float *shared_out, const float *weights, const float *shared_logit, uint32_t k,
                             uint32_t hidden, uint32_t tokens, float *y, float *routed, uint32_t *status, float *hc_residual,
                             const float *hc_inject, uint32_t hc_streams, void *stream);
extern "C" int qw4sh_build_groups(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream);
extern "C" int qw4sh_build_dense_groups(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream);

static int g_sm_count[64] = {0};
static int sm_count() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (!g_sm_count[device] && cudaDeviceGetAttribute(&g_sm_count[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        g_sm_count[device] = 148;
    return g_sm_count[device];
}
static int g_only_step = -1;                       // profiling: launch just one step of the layer (-1: all)
extern "C" void qw4sh_set_only_step(int step) { g_only_step = step; }
#define STEP(id) (g_only_step < 0 || g_only_step == (id))
static int g_expert_path = -1;                     // -1 auto, 0 CUDA-core kernels, 1 tensor-core grouped kernels
extern "C" void qw4sh_set_expert_path(int path) { g_expert_path = path; }

// Token batches up to this size take the decode path (groups of <= 4 rows on int8 MMA).
static const size_t MMA_MAX_TOKENS = 64;

static bool mma_path(const QW4ShLayer *layer, size_t tokens) {
    if (g_expert_path == 0) return false;
    if (g_expert_path < 0 && tokens > MMA_MAX_TOKENS) return false;
    return layer->w[1].type == layer->w[2].type && layer->w[4].type == layer->w[5].type &&
           qw4sh_mma_supported(&layer->w[1], 0) && qw4sh_mma_supported(&layer->w[2], 0) && qw4sh_mma_supported(&layer->w[3], 1) &&
           qw4sh_mma_supported(&layer->w[4], 0) && qw4sh_mma_supported(&layer->w[5], 0) && qw4sh_mma_supported(&layer->w[6], 1);
}

// Batches of more than MMA_MAX_TOKENS rows take the tcgen05 prefill kernels when every expert tensor is Q4_K.
static int g_prefill_path = -1;                    // -1 automatic, 0 never
extern "C" void qw4sh_set_prefill_path(int path) { g_prefill_path = path; }
static bool prefill_path(const QW4ShLayer *layer, size_t tokens) {
    if (g_prefill_path == 0 || g_expert_path == 0 || tokens <= MMA_MAX_TOKENS) return false;
    for (int i = 1; i <= 6; i++) if (!qw4sh_prefill_supported(&layer->w[i], i == 3 || i == 6)) return false;
    return layer->inter % 32 == 0 && layer->shared_inter % 32 == 0;
}

// Batches of more than four rows (and any batch the one-kernel decode or the tcgen05 prefill cannot take) run the
// expert products on the tile kernels: weight fragments built once per 32-row group instead of once per 4 rows.
static int g_tile_path = -1;                       // -1 automatic, 0 never, 1 whenever the types allow
extern "C" void qw4sh_set_tile_path(int path) { g_tile_path = path; }
static bool tile_types(const QW4ShLayer *layer) {
    return layer->w[1].type == layer->w[2].type && qw4sh_tile_supported(&layer->w[1], 0) && qw4sh_tile_supported(&layer->w[2], 0) &&
           qw4sh_tile_supported(&layer->w[3], 1);
}
static bool tile_path(const QW4ShLayer *layer, size_t tokens) {
    if (g_tile_path == 0 || g_expert_path == 0 || (g_tile_path > 0 && tokens <= 4)) return false;
    // automatic: batches that neither the four-row kernels (<= 64 rows, Q4_K / IQ2_XXS) nor the tcgen05 prefill
    // (Q4_K) can take: IQ2_XXS beyond 64 rows, Q2_K at any size; 1: every batch of more than four rows
    if (g_tile_path < 0 && (tokens <= MMA_MAX_TOKENS ? mma_path(layer, tokens) : prefill_path(layer, tokens))) return false;
    return tile_types(layer) && layer->w[4].type == layer->w[5].type && qw4sh_tile_supported(&layer->w[4], 0) &&
           qw4sh_tile_supported(&layer->w[5], 0) && qw4sh_tile_supported(&layer->w[6], 1);
}

static cudaStream_t g_side_stream[64] = {nullptr};
static cudaEvent_t g_side_event[64][4] = {{nullptr}};
static int side_stream(cudaStream_t *stream, cudaEvent_t **events) {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(cudaErrorInvalidDevice, "device index");
    if (!g_side_stream[device]) {
        CU(cudaStreamCreateWithFlags(&g_side_stream[device], cudaStreamNonBlocking));
        for (int i = 0; i < 4; i++) CU(cudaEventCreateWithFlags(&g_side_event[device][i], cudaEventDisableTiming));
    }
    *stream = g_side_stream[device]; *events = g_side_event[device];
    return 0;
}

// A third stream, for work of the expert-parallel step that may run beside both the main stream and the shared
// expert's branch (the digits of the gathered rows, beside the lists): stream and two events, [0] fork, [1] done.
static cudaStream_t g_aux_stream[64] = {nullptr};
static cudaEvent_t g_aux_event[64][2] = {{nullptr}};
static int aux_stream(cudaStream_t *stream, cudaEvent_t **events) {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(cudaErrorInvalidDevice, "device index");
    if (!g_aux_stream[device]) {
        CU(cudaStreamCreateWithFlags(&g_aux_stream[device], cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++) CU(cudaEventCreateWithFlags(&g_aux_event[device][i], cudaEventDisableTiming));
    }
    *stream = g_aux_stream[device]; *events = g_aux_event[device];
    return 0;
}

static int launch_route_group_small(const QW4ShLayer *layer, const QW4ShWork *work, uint32_t T, cudaStream_t stream) {
    const uint32_t E = layer->experts, k = layer->top_k;
    route_group_small_kernel<<<T, 512, (size_t)T * k * 4, stream>>>(E, k, layer->norm, work->logits, T, work->probs, work->ids,
                                                                    work->weights, work->offsets, work->pair_to_row, work->row_to_pair,
                                                                    work->active, (Group4 *)work->groups, work->n_groups, work->status);
    LAUNCHED("route_group_small_kernel");
    return 0;
}

static bool takes_fused(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, const float *y, size_t tokens) {
    return g_only_step < 0 && g_expert_path != 0 && !work->routed && qw4sh_fused_supported(layer, tokens, x, y, sm_count());
}

// Whether a forward of this batch would run as the one-kernel decode path (which writes every y element exactly once
// and never reads y, so y may lie in pinned host memory).
extern "C" int qw4sh_takes_fused(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, const float *y, size_t tokens) {
    return !g_stage_timing && takes_fused(layer, work, x, y, tokens) ? 1 : 0;
}

__global__ void __launch_bounds__(256) hc_add_kernel(const float *__restrict__ y, uint32_t hidden, HcAdd hc, uint32_t *status) {
    const uint32_t t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c < hidden && !hc_add(hc, t, c, hidden, y[(uint64_t)t * hidden + c])) atomicOr(status, QW4SH_ERR_NONFINITE);
}

static int layer_launches(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens,
                          uint32_t *ids_out, float *weights_out, int router_mode, bool timed) {
    cudaStream_t stream = (cudaStream_t)work->stream;
    const uint32_t T = (uint32_t)tokens, k = layer->top_k, E = layer->experts, H = layer->hidden;
    if (!timed && takes_fused(layer, work, x, y, tokens)) {
        // a cooperative grid that cannot be resident all at once (another context holds SMs) is refused
        // at launch: the multi-kernel sequence below does the same work
        const int fused_rc = qw4sh_fused_decode(layer, work, x, y, tokens, ids_out, weights_out, router_mode, sm_count());
        if (fused_rc != (int)cudaErrorCooperativeLaunchTooLarge) return fused_rc;
        (void)cudaGetLastError();
    }
    const bool tile = tile_path(layer, tokens);
    const bool mma = tile || mma_path(layer, tokens);
    const bool fused_route = mma && T <= 64 && E <= 512 && k <= E && T * k < 4096;
    int rc, stage = 0;
#define STAGE_MARK() do { if (timed) CU(cudaEventRecord(g_stage_event[stage++], stream)); } while (0)
    STAGE_MARK();
    // The shared expert and the quantisation of x need only x: they run on a second stream
    // beside router and route, and join before the routed experts / the combine.  (Serial when
    // timing stages.)
    cudaStream_t side = stream;
    cudaEvent_t *ev = nullptr;                          // [0] fork, [1] x digits ready, [2] routes ready, [3] shared expert done
    const bool overlap = mma && !timed;
    uint8_t *shared_groups = (uint8_t *)work->groups + (size_t)T * k * 16;      // behind the routed groups
    if (overlap) {
        if ((rc = side_stream(&side, &ev))) return rc;
        CU(cudaEventRecord(ev[0], stream));
        CU(cudaStreamWaitEvent(side, ev[0], 0));
    }
    if (mma) {
        if (STEP(1) && (rc = qw4sh_quantize_rows(x, T, H, work->xq, work->xneg, work->xsum, work->xscale, side))) return rc;
        if (overlap) CU(cudaEventRecord(ev[1], side));
    }
    const int ctas = sm_count();
    // expert products of one stage: tile kernels over groups of <= 32 rows, or the 4-row grouped kernel
    auto products = [&](int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, bool shared, const uint32_t *r2p, uint32_t k_div, const int8_t *q,
                        const int8_t *neg, const int *sums, const float *scale, float *out, cudaStream_t strm) -> int {
        if (tile)
            return qw4sh_expert_tiles(mode, w0, w1, shared ? (void *)shared_groups : work->groups, work->n_groups + (shared ? 1 : 0), r2p, k_div,
                                      q, sums, scale, out, work->status, ctas, strm);
        return qw4sh_grouped_mma(mode, w0, w1, shared ? (void *)shared_groups : work->groups, work->n_groups + (shared ? 1 : 0), r2p, k_div, q, neg,
                                 sums, scale, out, work->status, ctas, strm);
    };
    auto shared_branch = [&](int which) -> int {
        if (which == 0) {
            if (tile) { if ((rc = qw4sh_build_dense_tile_groups(T, shared_groups, work->n_groups + 1, side))) return rc; }
            else if (!fused_route && (rc = qw4sh_build_dense_groups(T, shared_groups, work->n_groups + 1, side))) return rc;
            if (!STEP(4)) return 0;
            return products(0, &layer->w[4], &layer->w[5], true, nullptr, 1, work->xq, work->xneg, work->xsum, work->xscale, work->shared_act, side);
        }
        if (STEP(7) && (rc = qw4sh_quantize_rows(work->shared_act, T, layer->shared_inter, work->sq, work->sneg, work->ssum, work->sscale, side))) return rc;
        if (!STEP(8)) return 0;
        return products(1, &layer->w[6], nullptr, true, nullptr, 1, work->sq, work->sneg, work->ssum, work->sscale, work->shared_out, side);
    };
    if (STEP(0) && (rc = launch_router(layer, x, tokens, work->logits, work->shared_logit, work->status, router_mode, stream))) return rc;
    STAGE_MARK();
    if (fused_route) {
        if (STEP(2) && (rc = launch_route_group_small(layer, work, T, stream))) return rc;
        STAGE_MARK(); STAGE_MARK();
        if (overlap) {                                // shared groups are written by the fused kernel
            CU(cudaEventRecord(ev[2], stream));
            CU(cudaStreamWaitEvent(side, ev[2], 0));
        }
    } else {
        if ((rc = qw4sh_route(E, k, layer->norm, work->logits, E, tokens, work->probs, work->ids, work->weights, work->status, stream))) return rc;
        STAGE_MARK();
        if (tokens > 64 && work->dispatch_scratch) {
            if ((rc = qw4sh_group_large(E, k, tokens, work->ids, work->offsets, work->pair_to_row, work->row_to_pair, work->active,
                                        work->dispatch_scratch, work->status, stream))) return rc;
        } else if ((rc = qw4sh_group(E, k, tokens, work->ids, work->offsets, work->pair_to_row, work->row_to_pair, work->active, work->status, stream))) return rc;
        if (mma && !tile && (rc = qw4sh_build_groups(work->offsets, work->active, work->groups, work->n_groups, stream))) return rc;
        STAGE_MARK();
    }
    if (tile && (rc = qw4sh_build_tile_groups(work->offsets, work->active, work->groups, work->n_groups, stream))) return rc;
    if (mma) {
        if (overlap) {
            if ((rc = shared_branch(0)) || (rc = shared_branch(1))) return rc;
            CU(cudaEventRecord(ev[3], side));
            CU(cudaStreamWaitEvent(stream, ev[1], 0));
        }
        if (STEP(3) && (rc = products(0, &layer->w[1], &layer->w[2], false, work->row_to_pair, k, work->xq, work->xneg, work->xsum, work->xscale,
                                      work->act, stream))) return rc;
        STAGE_MARK();
        if (!overlap && (rc = shared_branch(0))) return rc;
        STAGE_MARK();
        if (STEP(5) && (rc = qw4sh_quantize_rows(work->act, T * k, layer->inter, work->aq, work->aneg, work->asum, work->ascale, stream))) return rc;
        if (STEP(6) && (rc = products(1, &layer->w[3], nullptr, false, work->row_to_pair, 1, work->aq, work->aneg, work->asum, work->ascale,
                                      work->out, stream))) return rc;
        STAGE_MARK();
        if (!overlap && (rc = shared_branch(1))) return rc;
        STAGE_MARK();
        if (overlap) CU(cudaStreamWaitEvent(stream, ev[3], 0));
        if (STEP(9) && (rc = qw4sh_combine(work->out, work->shared_out, work->weights, work->shared_logit, k, H, T, y, work->routed, work->status, work->hc_residual, work->hc_inject,
                                             work->hc_streams, stream))) return rc;
        STAGE_MARK();
    } else if (prefill_path(layer, tokens)) {
        // tensor-core prefill: groups of <= 32 rows, tcgen05 MMAs on exact integer codes.  (The shared expert on a second
        // stream beside router and dispatch was measured and made the step slower: its persistent CTAs hold every SM.)
        void *const *hf = work->half;
        if ((rc = qw4sh_build_groups32(work->offsets, work->active, work->groups32, work->n_groups32, stream))) return rc;
        if ((rc = qw4sh_build_dense_groups32(T, work->shared_groups32, work->n_groups32 + 1, stream))) return rc;
        if ((rc = qw4sh_split_rows(x, T, H, hf[0], hf[1], hf[2], hf[3], stream))) return rc;
        if ((rc = qw4sh_prefill_tc(0, &layer->w[1], &layer->w[2], work->groups32, work->n_groups32, work->row_to_pair, k, hf[0], hf[1], hf[2],
                                   hf[3], hf[4], hf[5], hf[6], hf[7], nullptr, work->status, ctas, stream))) return rc;
        STAGE_MARK();
        if ((rc = qw4sh_prefill_tc(0, &layer->w[4], &layer->w[5], work->shared_groups32, work->n_groups32 + 1, nullptr, 1, hf[0], hf[1], hf[2],
                                   hf[3], hf[8], hf[9], hf[10], hf[11], nullptr, work->status, ctas, stream))) return rc;
        STAGE_MARK();
        if ((rc = qw4sh_prefill_tc(1, &layer->w[3], nullptr, work->groups32, work->n_groups32, work->row_to_pair, 1, hf[4], hf[5], hf[6], hf[7],
                                   nullptr, nullptr, nullptr, nullptr, work->out, work->status, ctas, stream))) return rc;
        STAGE_MARK();
        if ((rc = qw4sh_prefill_tc(1, &layer->w[6], nullptr, work->shared_groups32, work->n_groups32 + 1, nullptr, 1, hf[8], hf[9], hf[10],
                                   hf[11], nullptr, nullptr, nullptr, nullptr, work->shared_out, work->status, ctas, stream))) return rc;
        STAGE_MARK();
        if ((rc = qw4sh_combine(work->out, work->shared_out, work->weights, work->shared_logit, k, H, T, y, work->routed, work->status, work->hc_residual, work->hc_inject,
                                             work->hc_streams, stream))) return rc;
        STAGE_MARK();
    } else {
        const uint32_t groups = (uint32_t)(tokens * k < E ? tokens * k : E);
        if ((rc = launch_gate_up(as_dev(layer->w[1]), as_dev(layer->w[2]), x, H, work->offsets, work->row_to_pair, work->active, k, T,
                                 groups, work->act, work->status, stream))) return rc;
        STAGE_MARK();
        if ((rc = launch_gate_up(as_dev(layer->w[4]), as_dev(layer->w[5]), x, H, nullptr, nullptr, nullptr, 1, T, 1,
                                 work->shared_act, work->status, stream))) return rc;
        STAGE_MARK();
        if ((rc = launch_down(as_dev(layer->w[3]), as_dev(layer->w[6]), work->act, work->shared_act, work->ids, work->weights,
                              work->shared_logit, k, T, y, work->routed, work->status, stream))) return rc;
        if (work->hc_residual) {                      // the CUDA-core kernels are the fallback for every format: the add follows as a kernel of its own
            hc_add_kernel<<<dim3((H + 255) / 256, T), 256, 0, stream>>>(y, H, HcAdd{work->hc_residual, work->hc_inject, work->hc_streams}, work->status);
            LAUNCHED("hc_add_kernel");
        }
        STAGE_MARK(); STAGE_MARK(); STAGE_MARK();
    }
#undef STAGE_MARK
    if (ids_out || weights_out) {
        copy_routes_kernel<<<(T * k + 255) / 256, 256, 0, stream>>>(work->ids, work->weights, T * k, ids_out, weights_out);
        LAUNCHED("copy_routes_kernel");
    }
    return 0;
}

// ------------------------------------------------------------------------------------
// Pieces of the layer that run on their own.
// ------------------------------------------------------------------------------------
extern "C" int qw4sh_group_rows(uint32_t experts, size_t rows, const uint32_t *ids, uint32_t *offsets, uint32_t *pair_to_row,
                                uint32_t *row_to_pair, uint32_t *active, uint32_t *status, void *stream) {
    if (!rows) return 0;
    if (experts > 1024 || rows >= (1u << 20)) return fail(cudaErrorInvalidValue, "row dispatch: at most 1024 experts and 2^20 rows");
    group_rows_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(experts, (uint32_t)rows, ids, offsets, pair_to_row, row_to_pair, active, status);
    LAUNCHED("group_rows_kernel");
    return 0;
}

extern "C" int qw4sh_route_forward(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, size_t tokens, int router_mode) {
    if (!tokens) return 0;
    if (ensure_constants()) return -1;
    cudaStream_t stream = (cudaStream_t)work->stream;
    int rc;
    if ((rc = launch_router(layer, x, tokens, work->logits, work->shared_logit, work->status, router_mode, stream))) return rc;
    return qw4sh_route(layer->experts, layer->top_k, layer->norm, work->logits, layer->experts, tokens, work->probs, work->ids,
                       work->weights, work->status, stream);
}

// ---- expert parallelism (ep_nccl.cu holds the exchange) -------------------------------------------------
extern "C" uint32_t qw4sh_ep_row_floats(uint32_t hidden, uint32_t k);
extern "C" int qw4sh_ep_pack_rows(const float *x, const uint32_t *ids, const float *weights, uint32_t tokens, uint32_t hidden, uint32_t k,
                                  float *msg, void *stream);
extern "C" int qw4sh_ep_local_ids(const float *msg, uint32_t hidden, uint32_t k, uint32_t tokens, uint32_t experts, uint32_t first,
                                  uint32_t count, uint32_t *local, uint32_t *status, void *stream);
extern "C" int qw4sh_ep_partial(const float *msg, uint32_t hidden, uint32_t k, uint32_t tokens, const uint32_t *local, const float *out,
                                const float *shared_out, const float *shared_logit, uint32_t own_first, uint32_t own, float *partial,
                                uint32_t *status, void *stream);
extern "C" int qw4sh_quantize_rows_listed(const float *x, uint32_t pitch, uint32_t max_rows, uint32_t k, const uint32_t *row_list,
                                          const uint32_t *row_begin, const uint32_t *row_end, int8_t *xq, int8_t *xneg, int *xsum, float *xscale,
                                          void *stream);
extern "C" int qw4sh_ep_active_slice(const uint32_t *active, uint32_t first, uint32_t count, uint32_t *active_local, void *stream);

// Per-stage timing of the expert-parallel step (profiling aid): with the trace on, an event is recorded at every
// stage boundary and the step ends with a synchronisation that adds the stage times up.
enum { EP_STAGES = 10 };
static int g_ep_trace = 0;
static cudaEvent_t g_ep_event[EP_STAGES + 1] = {nullptr};
static double g_ep_ms[EP_STAGES] = {0};
static uint64_t g_ep_steps = 0;
extern "C" void qw4sh_ep_trace(int on) {
    g_ep_trace = on ? 1 : 0;
    for (int i = 0; i < EP_STAGES; i++) g_ep_ms[i] = 0;
    g_ep_steps = 0;
}
extern "C" int qw4sh_ep_trace_on(void) { return g_ep_trace; }
extern "C" int qw4sh_ep_trace_mark(int index, void *stream) {
    if (!g_ep_trace || index < 0 || index > EP_STAGES) return 0;
    if (!g_ep_event[index]) CU(cudaEventCreate(&g_ep_event[index]));
    CU(cudaEventRecord(g_ep_event[index], (cudaStream_t)stream));
    return 0;
}
// After the last mark of a step: waits and accumulates (stage i = mark i .. mark i + 1).
extern "C" int qw4sh_ep_trace_collect(void) {
    if (!g_ep_trace) return 0;
    CU(cudaEventSynchronize(g_ep_event[EP_STAGES]));
    for (int i = 0; i < EP_STAGES; i++) {
        float ms = 0.0f;
        if (g_ep_event[i] && g_ep_event[i + 1] && cudaEventElapsedTime(&ms, g_ep_event[i], g_ep_event[i + 1]) == cudaSuccess) g_ep_ms[i] += ms;
    }
    g_ep_steps++;
    return 0;
}
extern "C" uint64_t qw4sh_ep_trace_read(double *ms, int n) {
    for (int i = 0; i < n && i < EP_STAGES; i++) ms[i] = g_ep_ms[i];
    return g_ep_steps;
}

static bool shared_on_mma(const QW4ShLayer *layer) {
    return layer->w[4].type == layer->w[5].type && qw4sh_mma_supported(&layer->w[4], 0) && qw4sh_mma_supported(&layer->w[5], 0) &&
           qw4sh_mma_supported(&layer->w[6], 1);
}
static bool shared_on_tiles(const QW4ShLayer *layer) {
    return layer->w[4].type == layer->w[5].type && qw4sh_tile_supported(&layer->w[4], 0) && qw4sh_tile_supported(&layer->w[5], 0) &&
           qw4sh_tile_supported(&layer->w[6], 1);
}

// The shared expert of `tokens` own tokens, on the side stream: it needs only x, so it runs under the exchange.
// Its x digits live in the LAST rows of the quantisation buffers (rows 0 .. total-1 belong to the gathered rows).
static int ep_shared_begin(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, size_t tokens) {
    if (!tokens) return 0;
    const bool tiles = tokens > MMA_MAX_TOKENS || !shared_on_mma(layer);
    if (tiles ? !shared_on_tiles(layer) : !shared_on_mma(layer))
        return fail(cudaErrorNotSupported, "expert-parallel step needs a Q4_K, IQ2_XXS or Q2_K shared expert");
    cudaStream_t stream = (cudaStream_t)work->stream, side;
    cudaEvent_t *ev;
    int rc;
    if ((rc = side_stream(&side, &ev))) return rc;
    const uint32_t T = (uint32_t)tokens, H = layer->hidden;
    const size_t off = work->cap - tokens;
    int8_t *xq = work->xq + off * 2 * H, *xneg = work->xneg + off * 2 * H;
    int *xsum = work->xsum + off * (H / 32) * 2;
    float *xscale = work->xscale + off;
    const int ctas = sm_count();
    CU(cudaEventRecord(ev[0], stream));
    CU(cudaStreamWaitEvent(side, ev[0], 0));
    if ((rc = qw4sh_quantize_rows(x, T, H, xq, xneg, xsum, xscale, side))) return rc;
    if (tiles) {
        if ((rc = qw4sh_build_dense_tile_groups(T, work->shared_groups, work->n_groups + 3, side))) return rc;
        if ((rc = qw4sh_expert_tiles(0, &layer->w[4], &layer->w[5], work->shared_groups, work->n_groups + 3, nullptr, 1, xq, xsum, xscale,
                                     work->shared_act, work->status, ctas, side))) return rc;
        if ((rc = qw4sh_quantize_rows(work->shared_act, T, layer->shared_inter, work->sq, work->sneg, work->ssum, work->sscale, side))) return rc;
        if ((rc = qw4sh_expert_tiles(1, &layer->w[6], nullptr, work->shared_groups, work->n_groups + 3, nullptr, 1, work->sq, work->ssum,
                                     work->sscale, work->shared_out, work->status, ctas, side))) return rc;
    } else {
        if ((rc = qw4sh_build_dense_groups(T, work->shared_groups, work->n_groups + 3, side))) return rc;
        if ((rc = qw4sh_grouped_mma(0, &layer->w[4], &layer->w[5], work->shared_groups, work->n_groups + 3, nullptr, 1, xq, xneg, xsum, xscale,
                                    work->shared_act, work->status, ctas, side))) return rc;
        if ((rc = qw4sh_quantize_rows(work->shared_act, T, layer->shared_inter, work->sq, work->sneg, work->ssum, work->sscale, side))) return rc;
        if ((rc = qw4sh_grouped_mma(1, &layer->w[6], nullptr, work->shared_groups, work->n_groups + 3, nullptr, 1, work->sq, work->sneg, work->ssum,
                                    work->sscale, work->shared_out, work->status, ctas, side))) return rc;
    }
    CU(cudaEventRecord(ev[3], side));
    return 0;
}

// Step 1 of an expert-parallel layer on this rank: router and routes of its own tokens, the exchange rows
// packed into msg_local, the shared expert started beside.
extern "C" int qw4sh_ep_begin(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, size_t tokens, float *msg_local, int router_mode) {
    if (!tokens) return 0;
    int rc;
    if ((rc = qw4sh_ep_trace_mark(0, work->stream))) return rc;
    if ((rc = launch_router(layer, x, tokens, work->logits, work->shared_logit, work->status, router_mode, (cudaStream_t)work->stream))) return rc;
    if ((rc = qw4sh_ep_trace_mark(1, work->stream))) return rc;
    if ((rc = qw4sh_route(layer->experts, layer->top_k, layer->norm, work->logits, layer->experts, tokens, work->probs, work->ids, work->weights,
                          work->status, work->stream))) return rc;
    if ((rc = qw4sh_ep_pack_rows(x, work->ids, work->weights, (uint32_t)tokens, layer->hidden, layer->top_k, msg_local, work->stream))) return rc;
    if ((rc = qw4sh_ep_trace_mark(2, work->stream))) return rc;
    return ep_shared_begin(layer, work, x, tokens);
}

// Step 3: this rank's experts (global ids first_expert .. + local_experts) over the gathered rows of `total` tokens,
// then the per-token partial sums; tokens [own_first, own_first + own) are this rank's (they get the shared expert).
extern "C" int qw4sh_ep_experts(const QW4ShLayer *layer, const QW4ShWork *work, const float *msg_all, size_t total, size_t own_first, size_t own,
                                uint32_t first_expert, uint32_t local_experts, float *partial) {
    if (!total) return 0;
    if (ensure_constants()) return -1;
    if (total + own > work->cap) return fail(cudaErrorInvalidValue, "workspace too small: capacity must cover all ranks' tokens plus its own");
    cudaStream_t stream = (cudaStream_t)work->stream;
    const uint32_t T = (uint32_t)total, H = layer->hidden, k = layer->top_k, pitch = qw4sh_ep_row_floats(H, k);
    uint32_t *local = work->ids + own * k;                                  // behind this rank's own routes
    int rc;
    if ((rc = qw4sh_ep_trace_mark(3, stream))) return rc;                   // stage 2 was the all-gather
    // the digits of the gathered rows depend on the rows alone: they are made on a stream of their own beside the lists
    // (in one stream, as before, while stages are being timed)
    cudaStream_t aux = stream;
    cudaEvent_t *aux_ev = nullptr;
    const bool beside = !qw4sh_ep_trace_on();
    if (beside) {
        if ((rc = aux_stream(&aux, &aux_ev))) return rc;
        CU(cudaEventRecord(aux_ev[0], stream));
        CU(cudaStreamWaitEvent(aux, aux_ev[0], 0));
        if ((rc = qw4sh_quantize_rows_pitched(msg_all, pitch, T, H, work->xq, work->xneg, work->xsum, work->xscale, aux))) return rc;
        CU(cudaEventRecord(aux_ev[1], aux));
    }
    // Lists.  Small batches: the foreign ids are masked out and one CTA sorts the rest.  Large batches: the bitmap
    // dispatch sorts ALL pairs by global expert (a token meets an expert at most once), and this rank's experts are a
    // contiguous slice of that order: its offsets start at offsets[first_expert], its rows at row_to_pair[that].
    const bool sliced = (size_t)T * k > 2048 && work->dispatch_scratch && first_expert + local_experts <= layer->experts;
    const uint32_t *offsets = work->offsets, *active = work->active, *row_begin = nullptr;
    if (sliced) {
        if ((rc = qw4sh_ep_local_ids(msg_all, H, k, T, layer->experts, 0, layer->experts, local, work->status, stream))) return rc;   // global ids, dense
        if ((rc = qw4sh_group_large(layer->experts, k, T, local, work->offsets, work->pair_to_row, work->row_to_pair, work->active,
                                    work->dispatch_scratch, work->status, stream))) return rc;
        uint32_t *active_local = work->dispatch_scratch;                     // the bitmaps are dead after the placement
        if ((rc = qw4sh_ep_active_slice(work->active, first_expert, local_experts, active_local, stream))) return rc;
        offsets = work->offsets + first_expert; active = active_local; row_begin = offsets;
        if ((rc = qw4sh_ep_local_ids(msg_all, H, k, T, layer->experts, first_expert, local_experts, local, work->status, stream))) return rc;
    } else {
        if ((rc = qw4sh_ep_local_ids(msg_all, H, k, T, layer->experts, first_expert, local_experts, local, work->status, stream))) return rc;
        if ((rc = qw4sh_group_rows(local_experts, (size_t)T * k, local, work->offsets, work->pair_to_row, work->row_to_pair, work->active,
                                   work->status, stream))) return rc;
    }
    const bool mma_types = layer->w[1].type == layer->w[2].type && qw4sh_mma_supported(&layer->w[1], 0) && qw4sh_mma_supported(&layer->w[2], 0) &&
                           qw4sh_mma_supported(&layer->w[3], 1);
    const bool tiles = g_tile_path != 0 && tile_types(layer) && (g_tile_path > 0 || !mma_types || total > MMA_MAX_TOKENS);
    if (!tiles && !mma_types) return fail(cudaErrorNotSupported, "expert-parallel step needs Q4_K, IQ2_XXS or Q2_K expert tensors");
    const int ctas = sm_count();
    const uint32_t *row_end = offsets + local_experts;                      // rows of this rank's experts: [*row_begin (or 0), *row_end)
    if ((rc = qw4sh_ep_trace_mark(4, stream))) return rc;
    if (beside) CU(cudaStreamWaitEvent(stream, aux_ev[1], 0));
    else if ((rc = qw4sh_quantize_rows_pitched(msg_all, pitch, T, H, work->xq, work->xneg, work->xsum, work->xscale, stream))) return rc;
    if ((rc = qw4sh_ep_trace_mark(5, stream))) return rc;
    if (tiles) {
        if ((rc = qw4sh_build_tile_groups(offsets, active, work->groups, work->n_groups, stream))) return rc;
        if ((rc = qw4sh_expert_tiles(0, &layer->w[1], &layer->w[2], work->groups, work->n_groups, work->row_to_pair, k, work->xq, work->xsum,
                                     work->xscale, work->act, work->status, ctas, stream))) return rc;
        if ((rc = qw4sh_ep_trace_mark(6, stream))) return rc;
        if ((rc = qw4sh_quantize_rows_listed(work->act, layer->inter, T * k, layer->inter, work->row_to_pair, row_begin, row_end, work->aq, work->aneg,
                                             work->asum, work->ascale, stream))) return rc;
        if ((rc = qw4sh_ep_trace_mark(7, stream))) return rc;
        if ((rc = qw4sh_expert_tiles(1, &layer->w[3], nullptr, work->groups, work->n_groups, work->row_to_pair, 1, work->aq, work->asum,
                                     work->ascale, work->out, work->status, ctas, stream))) return rc;
    } else {
        if ((rc = qw4sh_build_groups(offsets, active, work->groups, work->n_groups, stream))) return rc;
        if ((rc = qw4sh_grouped_mma(0, &layer->w[1], &layer->w[2], work->groups, work->n_groups, work->row_to_pair, k, work->xq, work->xneg,
                                    work->xsum, work->xscale, work->act, work->status, ctas, stream))) return rc;
        if ((rc = qw4sh_ep_trace_mark(6, stream))) return rc;
        if ((rc = qw4sh_quantize_rows_listed(work->act, layer->inter, T * k, layer->inter, work->row_to_pair, row_begin, row_end, work->aq, work->aneg,
                                             work->asum, work->ascale, stream))) return rc;
        if ((rc = qw4sh_ep_trace_mark(7, stream))) return rc;
        if ((rc = qw4sh_grouped_mma(1, &layer->w[3], nullptr, work->groups, work->n_groups, work->row_to_pair, 1, work->aq, work->aneg,
                                    work->asum, work->ascale, work->out, work->status, ctas, stream))) return rc;
    }
    if ((rc = qw4sh_ep_trace_mark(8, stream))) return rc;
    if (own) {
        cudaStream_t side; cudaEvent_t *ev;
        if ((rc = side_stream(&side, &ev))) return rc;
        CU(cudaStreamWaitEvent(stream, ev[3], 0));
    }
    if ((rc = qw4sh_ep_partial(msg_all, H, k, T, local, work->out, work->shared_out, work->shared_logit, (uint32_t)own_first, (uint32_t)own, partial,
                               work->status, stream))) return rc;
    return qw4sh_ep_trace_mark(9, stream);                                  // stage 9 is the reduce-scatter
}

// The stream every workspace created afterwards (and every existing one, through
// qw4sh_current_stream) enqueues on.  nullptr: the library's own stream.
static cudaStream_t g_user_stream[64] = {nullptr};
static bool g_user_stream_set[64] = {false};
extern "C" int qw4sh_set_stream(void *stream) {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(cudaErrorInvalidDevice, "device index");
    g_user_stream[device] = (cudaStream_t)stream;
    g_user_stream_set[device] = stream != nullptr;
    return 0;
}
extern "C" int qw4sh_current_stream(void **stream) {
    int device = 0;
    CU(cudaGetDevice(&device));
    if (device >= 0 && device < 64 && g_user_stream_set[device]) { *stream = g_user_stream[device]; return 0; }
    return qw4sh_shared_stream(stream);
}

// The stream in force WITHOUT creating one: the caller's (qw4sh_set_stream), else the library's own if a
// workspace has already made it, else the legacy default stream (nullptr).
extern "C" int qw4sh_existing_stream(void **stream) {
    int device = 0;
    CU(cudaGetDevice(&device));
    *stream = nullptr;
    if (device < 0 || device >= 64) return fail(cudaErrorInvalidDevice, "device index");
    if (g_user_stream_set[device]) *stream = g_user_stream[device];
    else if (g_stream[device]) *stream = g_stream[device];
    return 0;
}
extern "C" int qw4sh_mem_info(size_t *free_bytes, size_t *total_bytes) {
    CU(cudaMemGetInfo(free_bytes, total_bytes));
    return 0;
}

extern "C" int qw4sh_fused_phase_clocks(const QW4ShWork *work, uint64_t clocks[16]) {
    CU(cudaMemcpy(clocks, work->sync + 8, 16 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return 0;
}
extern "C" int qw4sh_fused_repairs(const QW4ShWork *work, uint32_t *count) {
    CU(cudaMemcpy(count, work->sync + 48, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    return 0;
}

extern "C" int qw4sh_layer_forward(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens,
                                   uint32_t *ids_out, float *weights_out, int router_mode) {
    if (!tokens) return 0;
    if (ensure_constants()) return -1;
    cudaStream_t stream = (cudaStream_t)work->stream;
    if (g_stage_timing) {
        if (stage_collect()) return -1;
        for (int i = 0; i <= QW4SH_STAGES; i++) if (!g_stage_event[i]) CU(cudaEventCreate(&g_stage_event[i]));
        const int rc = layer_launches(layer, work, x, y, tokens, ids_out, weights_out, router_mode, true);
        g_stage_pending = rc == 0;
        return rc;
    }
    GraphCache *cache = (GraphCache *)work->graph_cache;
    // the one-kernel decode path is one launch already, chained to its neighbours by programmatic stream serialisation
    if (takes_fused(layer, work, x, y, tokens)) return layer_launches(layer, work, x, y, tokens, ids_out, weights_out, router_mode, false);
    if (!g_graph_mode || !cache) return layer_launches(layer, work, x, y, tokens, ids_out, weights_out, router_mode, false);
    if (work->hc_residual) return layer_launches(layer, work, x, y, tokens, ids_out, weights_out, router_mode, false);   // not replayed
    const bool same = cache->layer == layer && cache->x == x && cache->y == y && cache->ids == ids_out &&
                      cache->weights == weights_out && cache->tokens == tokens && cache->mode == router_mode;
    if (same && cache->exec) {
        CU(cudaGraphLaunch(cache->exec, stream));
        __sync_fetch_and_add(&g_launches, (unsigned long long)cache->seen);
        return 0;
    }
    if (!same) {                                      // first sight: run directly (also sets kernel attributes)
        if (cache->exec) { cudaGraphExecDestroy(cache->exec); cache->exec = nullptr; }
        cache->layer = layer; cache->x = x; cache->y = y; cache->ids = ids_out; cache->weights = weights_out;
        cache->tokens = tokens; cache->mode = router_mode;
        return layer_launches(layer, work, x, y, tokens, ids_out, weights_out, router_mode, false);
    }
    cudaGraph_t graph = nullptr;                      // second sight: capture, then replay
    const unsigned long long before = g_launches;
    CU(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    const int rc = layer_launches(layer, work, x, y, tokens, ids_out, weights_out, router_mode, false);
    cudaError_t e = cudaStreamEndCapture(stream, &graph);
    cache->seen = (int)(g_launches - before);
    g_launches = before;
    if (rc || e != cudaSuccess) { if (graph) cudaGraphDestroy(graph); return rc ? rc : fail(e, "graph capture"); }
    e = cudaGraphInstantiate(&cache->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { cache->exec = nullptr; return fail(e, "graph instantiate"); }
    CU(cudaGraphLaunch(cache->exec, stream));
    __sync_fetch_and_add(&g_launches, (unsigned long long)cache->seen);
    return 0;
}
