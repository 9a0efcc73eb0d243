// Expert products for decode-sized groups on the tensor cores (sm_100a).
//
// Work is cut into (group, row-tile) units.  A group is up to four token rows routed to one
// expert (larger per-expert lists are split into several groups by the dispatch kernel).
// Packed weights of a unit are staged into shared memory by TMA bulk copies
// (cp.async.bulk + mbarrier, a ring of stages fed by one producer warp), and sixteen consumer
// warps turn them into int8 MMA operands in registers:
//
//   Q4_K      the 4-bit codes ARE the A operand (nibbles masked out of the packed bytes);
//             sum(code * x) comes from mma.m16n8k32.s8, and the 6-bit sub-block scale and min
//             are applied to the int32 sums with integer multiply-adds
//   IQ2_XXS   the codebook vector (eight int8 magnitudes) comes from a bank-conflict-free
//             shared-memory table, signs are applied with one XOR per four weights and a
//             second MMA on the sign masks; the 4-bit group scale multiplies the int32 sums
//
// Activations enter as two int8 digits per value (x ~ dx * (q1 + q2 / 254), |error| <= dx/508
// with dx = max|x| / 127 per token), so four tokens fill the eight MMA columns and products
// are exact integers.  The fp16 super-scales are applied in FP32 once per half block.
//
// MMA k-slots are permuted so that each lane's eight k-slots of a 32-column chunk are eight
// CONSECUTIVE columns: lane (g, t) holds columns 8t..8t+7 of rows g and g+8, which is one
// codebook vector (IQ2_XXS) or eight code bytes (Q4_K), and one 64-bit read of the activation
// digits.
//
// Every wait on an mbarrier is bounded: after about a second the kernel records
// QW4SH_ERR_STATE, stops computing and runs out of its loops without hanging.
#include <cuda_runtime.h>
#include <stdint.h>

#include "cuda_shim.h"
#include "formats.cuh"

namespace qw4 {

constexpr int CW = 16;                          // consumer warps
constexpr int CT = CW * 32;                     // consumer threads
constexpr int NT = CT + 32;                     // + one producer warp
constexpr int TOK = 4;                          // token rows per group
constexpr uint32_t KMAX = 4096;                 // largest K held in shared memory

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false after ~1 s (2^31 SM cycles), with the error bit set.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *status) {
    if (mbar_try(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try(bar, parity)) {
        if (clock64() - start > (1ll << 31)) { atomicOr(status, QW4SH_ERR_STATE); return false; }
    }
    return true;
}
__device__ __forceinline__ void bulk_copy(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory"); }

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One group of the dispatch: rows [first, first + count) of the expert-sorted pair list.
struct VGroup { uint32_t expert, first, count, pad; };

struct GroupedArgs {
    DevTensor w0, w1;                  // gate and up, or down (w1 unused)
    const VGroup *groups;              // device list; n_groups[0] entries
    const uint32_t *n_groups;
    const uint32_t *row_to_pair;       // nullptr: pair = row (shared expert)
    uint32_t k_div;                    // token = pair / k_div for the gate/up input
    // gate_up input: activations prequantised per token by quantize_rows_kernel
    const int8_t *xq;                  // [tokens][2][K]
    const int *xsum;                   // [tokens][K/32][2] digit sums per 32-column chunk
    const float *xscale;               // [tokens] dx
    // down input: FP32 activations [pairs][K], quantised per group inside the CTA
    const float *act_in;
    float *out;                        // gate_up: act [pairs][n_out]; down: out [pairs][n_out]
    uint32_t *status;
};

template <uint32_t TYPE> struct Fmt;
template <> struct Fmt<T_Q4_K> {
    static constexpr uint32_t BLOCK_BYTES = 144;
    __host__ __device__ static uint32_t pitch(uint32_t nb) {           // row pitch = 8 words mod 32
        uint32_t p = nb * 144;
        while ((p / 4) % 32 != 8) p += 16;
        return p;
    }
    static constexpr bool NEEDS_LUT = false;
};
template <> struct Fmt<T_IQ2_XXS> {
    static constexpr uint32_t BLOCK_BYTES = 64;                          // payload; fp16 d kept apart
    __host__ __device__ static uint32_t pitch(uint32_t nb) {
        uint32_t p = nb * 64;
        while ((p / 4) % 32 != 8) p += 16;
        return p;
    }
    static constexpr bool NEEDS_LUT = true;
};

// Shared-memory plan (byte offsets), the same on host and device.
struct Plan {
    uint32_t bars, lut_grid, lut_sign, xq, xneg, xsum, tokmeta, partial, stages, stage_bytes, total;
    uint32_t n_stages, kp, pitch, unit_rows, matrices, dsec;
};
template <uint32_t TYPE, int MODE>
__host__ __device__ inline Plan make_plan(uint32_t k_storage) {
    Plan p;
    const uint32_t nb = k_storage / 256;
    p.unit_rows = MODE == 0 ? 16 : 64;
    p.matrices = MODE == 0 ? 2 : 1;
    p.kp = k_storage + 32;
    p.pitch = Fmt<TYPE>::pitch(nb);
    uint32_t at = 0;
    p.bars = at; at += 256;
    p.lut_grid = at; if (Fmt<TYPE>::NEEDS_LUT) at += 256 * 128;
    p.lut_sign = at; if (Fmt<TYPE>::NEEDS_LUT) at += 128 * 128;
    p.xq = at; at += 8 * p.kp;
    p.xneg = at; if (Fmt<TYPE>::NEEDS_LUT) at += 8 * p.kp;
    p.xsum = at; at += TOK * (k_storage / 32) * 8;
    p.tokmeta = at; at += 64;
    p.partial = at; at += 2 * CW * 32 * 2 * 4;                           // [parity][warp][64 floats]
    at = (at + 127) & ~127u;
    p.dsec = p.unit_rows * p.pitch;                                      // IQ2_XXS: fp16 d after the payload rows
    uint32_t per_matrix = p.unit_rows * p.pitch + (TYPE == T_IQ2_XXS ? ((p.unit_rows * nb * 2 + 15) & ~15u) : 0);
    per_matrix = (per_matrix + 127) & ~127u;
    p.stage_bytes = per_matrix * p.matrices;
    p.stages = at;
    const uint32_t budget = 200u * 1024u;
    uint32_t n = at < budget ? (budget - at) / p.stage_bytes : 0;
    p.n_stages = n > 8 ? 8 : n;
    p.total = at + p.n_stages * p.stage_bytes;
    return p;
}

// ------------------------------------------------------------------------------------
// Per-format consumption of one half block (128 columns = 4 chunks) for rows g and g+8.
// facc[0] += row g . x[token t], facc[1] += row g+8 . x[token t] (both still to be scaled by dx).
// ------------------------------------------------------------------------------------
template <uint32_t TYPE> struct Consume;

template <> struct Consume<T_Q4_K> {
    __device__ static __forceinline__ void half_block(const uint8_t *stage, const Plan &p, const uint8_t *smem, uint32_t nb,
                                                      uint32_t row0, uint32_t half, uint32_t g, uint32_t t, float (&facc)[2]) {
        const uint32_t b = half >> 1, hb = half & 1u;
        const uint8_t *r0 = stage + (row0 + g) * p.pitch + b * 144u, *r1 = r0 + 8 * p.pitch;
        const uint4 h0 = *reinterpret_cast<const uint4 *>(r0), h1 = *reinterpret_cast<const uint4 *>(r1);
        uint32_t sc0, mn0, sc1, mn1;
        if (hb == 0) { sc0 = h0.y & 0x3f3f3f3fu; mn0 = h0.z & 0x3f3f3f3fu; sc1 = h1.y & 0x3f3f3f3fu; mn1 = h1.z & 0x3f3f3f3fu; }
        else {
            sc0 = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u); mn0 = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u);
            sc1 = (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u); mn1 = ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u);
        }
        const uint8_t *xq = smem + p.xq + g * p.kp + (half * 4u) * 32u + 8u * t;
        const int2 *xsum = reinterpret_cast<const int2 *>(smem + p.xsum) + t * (nb * 8u) + half * 4u;
        int qacc[4] = {0, 0, 0, 0}, macc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {                                 // sub-block pair: low and high nibbles
            const uint2 q0 = *reinterpret_cast<const uint2 *>(r0 + 16 + (hb * 2 + cc) * 32 + 8 * t);
            const uint2 q1 = *reinterpret_cast<const uint2 *>(r1 + 16 + (hb * 2 + cc) * 32 + 8 * t);
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                const int j = cc * 2 + nib;                              // chunk within the half block
                const uint2 bq = *reinterpret_cast<const uint2 *>(xq + j * 32);
                int c[4] = {0, 0, 0, 0};
                mma_s8(c, (q0.x >> (4 * nib)) & 0x0f0f0f0fu, (q1.x >> (4 * nib)) & 0x0f0f0f0fu,
                       (q0.y >> (4 * nib)) & 0x0f0f0f0fu, (q1.y >> (4 * nib)) & 0x0f0f0f0fu, bq.x, bq.y);
                const int s0 = (int)((sc0 >> (8 * j)) & 0xffu), s1 = (int)((sc1 >> (8 * j)) & 0xffu);
                const int m0 = (int)((mn0 >> (8 * j)) & 0xffu), m1 = (int)((mn1 >> (8 * j)) & 0xffu);
                const int2 sx = xsum[j];
                qacc[0] += c[0] * s0; qacc[1] += c[1] * s0; qacc[2] += c[2] * s1; qacc[3] += c[3] * s1;
                macc[0] += sx.x * m0; macc[1] += sx.y * m0; macc[2] += sx.x * m1; macc[3] += sx.y * m1;
            }
        }
        const float lo = 1.0f / 254.0f;
        const float d0 = __half2float(__ushort_as_half((uint16_t)(h0.x & 0xffffu))), n0 = __half2float(__ushort_as_half((uint16_t)(h0.x >> 16)));
        const float d1 = __half2float(__ushort_as_half((uint16_t)(h1.x & 0xffffu))), n1 = __half2float(__ushort_as_half((uint16_t)(h1.x >> 16)));
        facc[0] += d0 * fmaf((float)qacc[1], lo, (float)qacc[0]) - n0 * fmaf((float)macc[1], lo, (float)macc[0]);
        facc[1] += d1 * fmaf((float)qacc[3], lo, (float)qacc[2]) - n1 * fmaf((float)macc[3], lo, (float)macc[2]);
    }
};

template <> struct Consume<T_IQ2_XXS> {
    __device__ static __forceinline__ void half_block(const uint8_t *stage, const Plan &p, const uint8_t *smem, uint32_t nb,
                                                      uint32_t row0, uint32_t half, uint32_t g, uint32_t t, float (&facc)[2]) {
        const uint32_t b = half >> 1, lane16 = (threadIdx.x & 15u) * 8u;
        const uint8_t *r0 = stage + (row0 + g) * p.pitch + half * 32u, *r1 = r0 + 8 * p.pitch;
        const uint8_t *grid = smem + p.lut_grid + lane16, *sign = smem + p.lut_sign + lane16;
        const uint8_t *xq = smem + p.xq + g * p.kp + (half * 4u) * 32u + 8u * t;
        const uint8_t *xn = smem + p.xneg + g * p.kp + (half * 4u) * 32u + 8u * t;
        int iacc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint2 g0 = *reinterpret_cast<const uint2 *>(r0 + 8 * j), g1 = *reinterpret_cast<const uint2 *>(r1 + 8 * j);
            const uint32_t i0 = (g0.x >> (8 * t)) & 0xffu, i1 = (g1.x >> (8 * t)) & 0xffu;
            const uint32_t s0 = (g0.y >> (7 * t)) & 127u, s1 = (g1.y >> (7 * t)) & 127u;
            const uint2 v0 = *reinterpret_cast<const uint2 *>(grid + i0 * 128u), v1 = *reinterpret_cast<const uint2 *>(grid + i1 * 128u);
            const uint2 m0 = *reinterpret_cast<const uint2 *>(sign + s0 * 128u), m1 = *reinterpret_cast<const uint2 *>(sign + s1 * 128u);
            const uint2 bq = *reinterpret_cast<const uint2 *>(xq + j * 32), bn = *reinterpret_cast<const uint2 *>(xn + j * 32);
            int c[4] = {0, 0, 0, 0};
            mma_s8(c, v0.x ^ m0.x, v1.x ^ m1.x, v0.y ^ m0.y, v1.y ^ m1.y, bq.x, bq.y);   // +v, or -v-1 where negative
            mma_s8(c, m0.x, m1.x, m0.y, m1.y, bn.x, bn.y);                                   // (-1) * (-x) adds the missing x
            const int w0 = (int)((g0.y >> 27) | 1u), w1 = (int)((g1.y >> 27) | 1u);         // 2 * scale + 1
            iacc[0] += c[0] * w0; iacc[1] += c[1] * w0; iacc[2] += c[2] * w1; iacc[3] += c[3] * w1;
        }
        const uint16_t *dsec = reinterpret_cast<const uint16_t *>(stage + p.dsec);
        const float d0 = __half2float(__ushort_as_half(dsec[(row0 + g) * nb + b])) * 0.125f;
        const float d1 = __half2float(__ushort_as_half(dsec[(row0 + g + 8) * nb + b])) * 0.125f;
        const float lo = 1.0f / 254.0f;
        facc[0] += d0 * fmaf((float)iacc[1], lo, (float)iacc[0]);
        facc[1] += d1 * fmaf((float)iacc[3], lo, (float)iacc[2]);
    }
};

// Producer: stage one unit (unit_rows rows of each matrix) with bulk copies.
template <uint32_t TYPE>
__device__ __forceinline__ void produce_unit(const GroupedArgs &a, const Plan &p, uint8_t *stage, uint64_t *full, uint32_t expert,
                                             uint32_t row0, uint32_t lane) {
    const uint32_t nb = a.w0.k_storage >> 8, rows = p.unit_rows;
    const uint32_t row_bytes = nb * Fmt<TYPE>::BLOCK_BYTES;
    const uint32_t dbytes = (rows * nb * 2 + 15) & ~15u;
    const uint32_t per_matrix = (rows * p.pitch + (TYPE == T_IQ2_XXS ? dbytes : 0) + 127) & ~127u;
    if (lane == 0) mbar_expect_tx(full, p.matrices * (rows * row_bytes + (TYPE == T_IQ2_XXS ? rows * nb * 2 : 0)));
    __syncwarp();
    for (uint32_t m = 0; m < p.matrices; m++) {
        const DevTensor &w = m == 0 ? a.w0 : a.w1;
        const uint8_t *mat = w.data + (uint64_t)expert * w.expert_bytes;
        uint8_t *dst = stage + m * per_matrix;
        for (uint32_t r = lane; r < rows; r += 32)
            bulk_copy(dst + r * p.pitch, mat + (uint64_t)(row0 + r) * row_bytes, row_bytes, full);
        if (TYPE == T_IQ2_XXS && lane == 0)
            bulk_copy(dst + p.dsec, mat + (uint64_t)w.n_out * nb * 64u + (uint64_t)row0 * nb * 2u, rows * nb * 2, full);
    }
}

// MODE 0: gate + up + SwiGLU -> act.  MODE 1: down -> out (one row per pair).
template <uint32_t TYPE, int MODE>
__global__ void __launch_bounds__(NT, 1) grouped_mma_kernel(const GroupedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t K = a.w0.k_storage, nb = K >> 8, halves = K >> 7;
    const Plan p = make_plan<TYPE, MODE>(K);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + p.bars), *empty = full + 8;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t n_groups = *a.n_groups;
    const uint32_t units_per_group = a.w0.n_out / p.unit_rows;
    const uint64_t total = (uint64_t)n_groups * units_per_group;
    const uint32_t u_begin = (uint32_t)(total * blockIdx.x / gridDim.x), u_end = (uint32_t)(total * (blockIdx.x + 1) / gridDim.x);

    if (tid == 0) {
        for (uint32_t s = 0; s < p.n_stages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (Fmt<TYPE>::NEEDS_LUT) {                                          // conflict-free tables: 16 copies, 8 B apart
        for (uint32_t i = tid; i < 256 * 16; i += NT) {
            const uint32_t entry = i >> 4, levels = c_iq2_levels[entry];
            uint32_t lo = 0, hi = 0;
            for (int j = 0; j < 4; j++) {
                lo |= iq2_magnitude((levels >> (2 * j)) & 3u) << (8 * j);
                hi |= iq2_magnitude((levels >> (2 * j + 8)) & 3u) << (8 * j);
            }
            *reinterpret_cast<uint2 *>(smem + p.lut_grid + entry * 128u + (i & 15u) * 8u) = make_uint2(lo, hi);
        }
        for (uint32_t i = tid; i < 128 * 16; i += NT) {
            const uint32_t signs = iq2_signs8(i >> 4);
            uint32_t lo = 0, hi = 0;
            for (int j = 0; j < 4; j++) {
                if ((signs >> j) & 1u) lo |= 0xffu << (8 * j);
                if ((signs >> (j + 4)) & 1u) hi |= 0xffu << (8 * j);
            }
            *reinterpret_cast<uint2 *>(smem + p.lut_sign + (i >> 4) * 128u + (i & 15u) * 8u) = make_uint2(lo, hi);
        }
    }
    __syncthreads();

    if (warp == CW) {                                                    // ---- producer warp ----
        uint32_t stage = 0, phase = 0;
        bool alive = true;
        for (uint32_t u = u_begin; u < u_end && alive; u++) {
            if (lane == 0 && u - u_begin >= p.n_stages) alive = mbar_wait(&empty[stage], phase ^ 1u, a.status);
            alive = __shfl_sync(0xffffffffu, alive, 0);
            if (!alive) break;
            const VGroup grp = a.groups[u / units_per_group];
            produce_unit<TYPE>(a, p, smem + p.stages + stage * p.stage_bytes, &full[stage], grp.expert,
                               (u % units_per_group) * p.unit_rows, lane);
            if (++stage == p.n_stages) { stage = 0; phase ^= 1u; }
        }
        return;
    }

    // ---- consumer warps ----
    const uint32_t g = lane >> 2, t = lane & 3u;
    uint32_t *tokmeta = reinterpret_cast<uint32_t *>(smem + p.tokmeta);  // [0..3] pair of token column, [4] count
    float *tokscale = reinterpret_cast<float *>(smem + p.tokmeta + 32);
    float *partial = reinterpret_cast<float *>(smem + p.partial);
    const uint32_t per_matrix = p.stage_bytes / p.matrices;
    uint32_t stage = 0, phase = 0, parity = 0, current = 0xffffffffu;
    bool alive = true;
    for (uint32_t u = u_begin; u < u_end; u++) {
        const uint32_t gi = u / units_per_group, row_tile = (u % units_per_group) * p.unit_rows;
        if (gi != current) {                                             // ---- stage this group's activations ----
            consumer_sync();
            const VGroup grp = a.groups[gi];
            if (tid < 8) {
                uint32_t pair = 0;
                if (tid < grp.count) pair = a.row_to_pair ? a.row_to_pair[grp.first + tid] : grp.first + tid;
                if (tid < TOK) tokmeta[tid] = pair;
                if (tid == 4) tokmeta[4] = grp.count;
            }
            if (MODE == 0) {
                for (uint32_t i = tid; i < TOK * 2 * (K >> 4); i += CT) {        // 16-byte pieces of the digit rows
                    const uint32_t col = i / (K >> 4), piece = i % (K >> 4), tok = col >> 1;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (tok < grp.count) {
                        const uint32_t pair = a.row_to_pair ? a.row_to_pair[grp.first + tok] : grp.first + tok;
                        v = *reinterpret_cast<const uint4 *>(a.xq + ((uint64_t)(pair / a.k_div) * 2 + (col & 1u)) * K + piece * 16);
                    }
                    *reinterpret_cast<uint4 *>(smem + p.xq + col * p.kp + piece * 16) = v;
                    if (Fmt<TYPE>::NEEDS_LUT)
                        *reinterpret_cast<uint4 *>(smem + p.xneg + col * p.kp + piece * 16) =
                            make_uint4(__vneg4(v.x), __vneg4(v.y), __vneg4(v.z), __vneg4(v.w));
                }
                for (uint32_t i = tid; i < TOK * (K >> 5); i += CT) {
                    const uint32_t tok = i / (K >> 5), chunk = i % (K >> 5);
                    int2 s = make_int2(0, 0);
                    if (tok < grp.count) {
                        const uint32_t pair = a.row_to_pair ? a.row_to_pair[grp.first + tok] : grp.first + tok;
                        s = *reinterpret_cast<const int2 *>(a.xsum + ((uint64_t)(pair / a.k_div) * (K >> 5) + chunk) * 2);
                    }
                    reinterpret_cast<int2 *>(smem + p.xsum)[i] = s;
                }
                if (tid < TOK) {
                    const uint32_t pair = tid < grp.count ? (a.row_to_pair ? a.row_to_pair[grp.first + tid] : grp.first + tid) : 0;
                    tokscale[tid] = tid < grp.count ? a.xscale[pair / a.k_div] : 0.0f;
                }
            } else {                                                     // quantise FP32 rows here (K <= 16 * CT)
                float *red = reinterpret_cast<float *>(smem + p.partial);      // reuse: [CW][TOK]
                float v[TOK][4];
                float amax[TOK];
#pragma unroll
                for (int r = 0; r < TOK; r++) {
                    amax[r] = 0.0f;
                    uint32_t pair = 0;
                    if ((uint32_t)r < grp.count) pair = a.row_to_pair ? a.row_to_pair[grp.first + r] : grp.first + r;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t col = tid + q * CT;
                        v[r][q] = ((uint32_t)r < grp.count && col < a.w0.k_logical) ? a.act_in[(uint64_t)pair * a.w0.k_logical + col] : 0.0f;
                        amax[r] = fmaxf(amax[r], fabsf(v[r][q]));
                    }
                    for (int o = 16; o; o >>= 1) amax[r] = fmaxf(amax[r], __shfl_xor_sync(0xffffffffu, amax[r], o));
                    if (lane == 0) red[warp * TOK + r] = amax[r];
                }
                consumer_sync();
#pragma unroll
                for (int r = 0; r < TOK; r++) {
                    float m = 0.0f;
                    for (int w = 0; w < CW; w++) m = fmaxf(m, red[w * TOK + r]);
                    const float dx = m > 0.0f ? m / 127.0f : 1.0f, inv = 1.0f / dx, inv2 = 254.0f / dx;
                    if (tid == 0) tokscale[r] = m > 0.0f ? dx : 0.0f;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t col = tid + q * CT;
                        if (col >= K) continue;
                        const float q1 = rintf(v[r][q] * inv);
                        const float q2 = fminf(fmaxf(rintf((v[r][q] - q1 * dx) * inv2), -127.0f), 127.0f);
                        const int i1 = (int)q1, i2 = (int)q2;
                        smem[p.xq + (2 * r) * p.kp + col] = (uint8_t)(int8_t)i1;
                        smem[p.xq + (2 * r + 1) * p.kp + col] = (uint8_t)(int8_t)i2;
                        if (Fmt<TYPE>::NEEDS_LUT) {
                            smem[p.xneg + (2 * r) * p.kp + col] = (uint8_t)(int8_t)(-i1);
                            smem[p.xneg + (2 * r + 1) * p.kp + col] = (uint8_t)(int8_t)(-i2);
                        }
                        int s1 = i1, s2 = i2;                            // warp = one 32-column chunk
                        for (int o = 16; o; o >>= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
                        if (lane == 0) reinterpret_cast<int2 *>(smem + p.xsum)[r * (K >> 5) + (col >> 5)] = make_int2(s1, s2);
                    }
                }
                consumer_sync();                                         // red[] is reused as partials below
            }
            consumer_sync();
            current = gi;
        }
        if (alive && lane == 0) alive = mbar_wait(&full[stage], phase, a.status);
        alive = __shfl_sync(0xffffffffu, alive, 0);
        const uint8_t *st = smem + p.stages + stage * p.stage_bytes;
        float facc[2] = {0.0f, 0.0f};
        uint32_t out_slot;
        if (MODE == 0) {                                                 // warp = (matrix, k-slice of 8)
            const uint32_t m = warp & 1u, ks = warp >> 1;
            if (alive)
                for (uint32_t h = ks; h < halves; h += 8) Consume<TYPE>::half_block(st + m * per_matrix, p, smem, nb, 0, h, g, t, facc);
            out_slot = warp;
        } else {                                                         // warp = (row tile of 4, k-slice of 4)
            const uint32_t rt = warp & 3u, ks = warp >> 2;
            if (alive)
                for (uint32_t h = ks; h < halves; h += 4) Consume<TYPE>::half_block(st, p, smem, nb, rt * 16, h, g, t, facc);
            out_slot = warp;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
        if (++stage == p.n_stages) { stage = 0; phase ^= 1u; }
        float *mine = partial + (parity * CW + out_slot) * 64;
        mine[lane] = facc[0];                                            // (row g, token t) at 4g + t
        mine[32 + lane] = facc[1];                                       // (row g + 8, token t)
        consumer_sync();
        const float *part = partial + parity * CW * 64;
        const uint32_t count = tokmeta[4];
        if (MODE == 0) {
            if (tid < 64) {                                              // 16 rows x 4 tokens
                const uint32_t row = tid >> 2, tok = tid & 3u;
                float gsum = 0.0f, usum = 0.0f;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) { gsum += part[(2 * ks) * 64 + tid]; usum += part[(2 * ks + 1) * 64 + tid]; }
                if (tok < count) {
                    const float dx = tokscale[tok];
                    gsum *= dx; usum *= dx;
                    const float e = __expf(-fabsf(gsum));
                    const float sig = gsum >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
                    const float v = gsum * sig * usum;
                    if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.out[(uint64_t)tokmeta[tok] * a.w0.n_out + row_tile + row] = v;
                }
            }
        } else {
            if (tid < 256) {                                             // 64 rows x 4 tokens
                const uint32_t rt = tid >> 6, within = tid & 63u, tok = within & 3u;
                float sum = 0.0f;
#pragma unroll
                for (int ks = 0; ks < 4; ks++) sum += part[(ks * 4 + rt) * 64 + within];
                if (tok < count) {
                    sum *= tokscale[tok];
                    if ((__float_as_uint(sum) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.out[(uint64_t)tokmeta[tok] * a.w0.n_out + row_tile + rt * 16 + (within >> 2)] = sum;
                }
            }
        }
        parity ^= 1u;
    }
}

// Two int8 digits per activation: x ~ dx * (q1 + q2 / 254), dx = max|x| / 127 per token.
// One CTA per token row.  Also writes the per-chunk digit sums Q4_K's min term needs.
__global__ void __launch_bounds__(512) quantize_rows_kernel(const float *__restrict__ x, uint32_t k, int8_t *__restrict__ xq,
                                                            int *__restrict__ xsum, float *__restrict__ xscale) {
    __shared__ float red[16];
    const uint32_t row = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float *src = x + (uint64_t)row * k;
    float amax = 0.0f;
    for (uint32_t c = tid; c < k; c += 512) amax = fmaxf(amax, fabsf(src[c]));
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < 16; w++) amax = fmaxf(amax, red[w]);
    const float dx = amax > 0.0f ? amax / 127.0f : 1.0f, inv = 1.0f / dx, inv2 = 254.0f / dx;
    if (tid == 0) xscale[row] = amax > 0.0f ? dx : 0.0f;
    for (uint32_t c = tid; c < k; c += 512) {                            // k is a multiple of 32: whole warps per chunk
        const float v = src[c], q1 = rintf(v * inv);
        const float q2 = fminf(fmaxf(rintf((v - q1 * dx) * inv2), -127.0f), 127.0f);
        int s1 = (int)q1, s2 = (int)q2;
        xq[((uint64_t)row * 2) * k + c] = (int8_t)s1;
        xq[((uint64_t)row * 2 + 1) * k + c] = (int8_t)s2;
        for (int o = 16; o; o >>= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
        if (lane == 0) { xsum[((uint64_t)row * (k >> 5) + (c >> 5)) * 2] = s1; xsum[((uint64_t)row * (k >> 5) + (c >> 5)) * 2 + 1] = s2; }
    }
}

// y[t, c] = sum over slots in slot order of weight[t, s] * out[t*k + s, c] + sigmoid(slogit[t]) * shared_out[t, c]
// (picoforge src/qwen4_moe.c:362-380).
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ out, const float *__restrict__ shared_out,
                                                      const float *__restrict__ weights, const float *__restrict__ shared_logit,
                                                      uint32_t k, uint32_t hidden, float *__restrict__ y, float *__restrict__ routed,
                                                      uint32_t *status) {
    const uint32_t t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= hidden) return;
    float sum = 0.0f;
    for (uint32_t s = 0; s < k; s++) sum = __fadd_rn(sum, __fmul_rn(weights[t * k + s], out[((uint64_t)t * k + s) * hidden + c]));
    const float sl = shared_logit[t], e = __expf(-fabsf(sl));
    const float gate = sl >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
    const float total = __fadd_rn(sum, __fmul_rn(gate, shared_out[(uint64_t)t * hidden + c]));
    if ((__float_as_uint(total) & 0x7f800000u) == 0x7f800000u || (__float_as_uint(sum) & 0x7f800000u) == 0x7f800000u)
        atomicOr(status, QW4SH_ERR_NONFINITE);
    if (routed) routed[(uint64_t)t * hidden + c] = sum;
    y[(uint64_t)t * hidden + c] = total;
}

// Groups of at most four rows out of the expert-sorted lists; one thread (lists are short).
__global__ void build_groups_kernel(const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ active, VGroup *groups,
                                    uint32_t *n_groups) {
    if (threadIdx.x || blockIdx.x) return;
    uint32_t n = 0;
    for (uint32_t i = 0; i < active[0]; i++) {
        const uint32_t e = active[1 + i], first = offsets[e], end = offsets[e + 1];
        for (uint32_t r = first; r < end; r += TOK) groups[n++] = VGroup{e, r, min((uint32_t)TOK, end - r), 0};
    }
    *n_groups = n;
}
__global__ void build_dense_groups_kernel(uint32_t tokens, VGroup *groups, uint32_t *n_groups) {
    const uint32_t n = (tokens + TOK - 1) / TOK;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        groups[i] = VGroup{0, i * TOK, min((uint32_t)TOK, tokens - i * TOK), 0};
    if (blockIdx.x == 0 && threadIdx.x == 0) *n_groups = n;
}

}  // namespace qw4

using namespace qw4;

extern "C" int qw4sh_note_launch(const char *name);      // kernels.cu: counts the launch, checks the error

static DevTensor dev(const QW4ShTensor &s) {
    DevTensor t;
    t.data = s.data; t.type = s.type; t.k_storage = s.k_storage; t.k_logical = s.k_logical;
    t.n_out = s.n_out; t.n_experts = s.n_experts; t.row_bytes = s.row_bytes; t.expert_bytes = s.expert_bytes;
    return t;
}

extern "C" int qw4sh_mma_supported(const QW4ShTensor *w, int mode) {
    if (w->type != T_Q4_K && w->type != T_IQ2_XXS) return 0;
    if (w->k_storage % 256 || w->k_storage > KMAX || w->k_logical != w->k_storage) return 0;
    if (w->n_out % (mode == 0 ? 16 : 64)) return 0;
    if (mode == 1 && w->k_storage > 4 * CT) return 0;
    return 1;
}

template <uint32_t TYPE, int MODE>
static int launch_grouped(const GroupedArgs &a, int ctas, cudaStream_t stream) {
    const Plan p = make_plan<TYPE, MODE>(a.w0.k_storage);
    if (p.n_stages < 2) return -2;
    cudaError_t e = cudaFuncSetAttribute(grouped_mma_kernel<TYPE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.total);
    if (e != cudaSuccess) return (int)e;
    grouped_mma_kernel<TYPE, MODE><<<ctas, NT, p.total, stream>>>(a);
    return qw4sh_note_launch("grouped_mma_kernel");
}

// mode 0: gate+up (w0, w1) -> out = act [pairs][n_out]; mode 1: down (w0) -> out [pairs][n_out].
extern "C" int qw4sh_grouped_mma(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                                 const uint32_t *row_to_pair, uint32_t k_div, const int8_t *xq, const int *xsum, const float *xscale,
                                 const float *act_in, float *out, uint32_t *status, int ctas, void *stream) {
    GroupedArgs a;
    a.w0 = dev(*w0); a.w1 = dev(w1 ? *w1 : *w0);
    a.groups = (const VGroup *)groups; a.n_groups = n_groups; a.row_to_pair = row_to_pair; a.k_div = k_div;
    a.xq = xq; a.xsum = xsum; a.xscale = xscale; a.act_in = act_in; a.out = out; a.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    if (w0->type == T_Q4_K) return mode == 0 ? launch_grouped<T_Q4_K, 0>(a, ctas, s) : launch_grouped<T_Q4_K, 1>(a, ctas, s);
    return mode == 0 ? launch_grouped<T_IQ2_XXS, 0>(a, ctas, s) : launch_grouped<T_IQ2_XXS, 1>(a, ctas, s);
}

extern "C" int qw4sh_quantize_rows(const float *x, uint32_t rows, uint32_t k, int8_t *xq, int *xsum, float *xscale, void *stream) {
    quantize_rows_kernel<<<rows, 512, 0, (cudaStream_t)stream>>>(x, k, xq, xsum, xscale);
    return qw4sh_note_launch("quantize_rows_kernel");
}
extern "C" int qw4sh_combine(const float *out, const float *shared_out, const float *weights, const float *shared_logit, uint32_t k,
                             uint32_t hidden, uint32_t tokens, float *y, float *routed, uint32_t *status, void *stream) {
    combine_kernel<<<dim3((hidden + 255) / 256, tokens), 256, 0, (cudaStream_t)stream>>>(out, shared_out, weights, shared_logit, k, hidden, y, routed, status);
    return qw4sh_note_launch("combine_kernel");
}
extern "C" int qw4sh_build_groups(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream) {
    build_groups_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(offsets, active, (VGroup *)groups, n_groups);
    return qw4sh_note_launch("build_groups_kernel");
}
extern "C" int qw4sh_build_dense_groups(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream) {
    build_dense_groups_kernel<<<(tokens / TOK + 256) / 256, 256, 0, (cudaStream_t)stream>>>(tokens, (VGroup *)groups, n_groups);
    return qw4sh_note_launch("build_dense_groups_kernel");
}
