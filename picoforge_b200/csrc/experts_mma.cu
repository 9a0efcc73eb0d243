// Expert products for decode-sized groups on the tensor cores (sm_100a).
//
// Work is cut into (group, row-tile) units.  A group is up to four token rows routed to one
// expert (larger per-expert lists are split into several groups by the dispatch kernel).
// One producer warp feeds two rings of shared-memory stages with TMA bulk copies
// (cp.async.bulk + mbarrier): packed weight rows of the next units, and the activation digits
// of the next group.  Sixteen consumer warps turn the packed bytes into int8 MMA operands in
// registers:
//
//   Q4_K      the 4-bit codes ARE the A operand (nibbles masked out of the packed bytes);
//             sum(code * x) comes from mma.m16n8k32.s8, and the 6-bit sub-block scale and min
//             are applied to the int32 sums with integer multiply-adds
//   IQ2_XXS   the codebook vector (eight int8 magnitudes) and the byte masks of its sign word
//             come from bank-conflict-free shared-memory tables; a negative weight is
//             (v ^ 0xff) + 1 per byte, two integer operations per four weights; the 4-bit
//             group scale multiplies the int32 sums
//
// Activations enter as two int8 digits per value (x ~ dx * (q1 + q2 / 254), |error| <= dx/508
// with dx = max|x| / 127 per row; quantize_rows_kernel), so four tokens fill the eight MMA
// columns and products are exact integers.  The fp16 super-scales are applied in FP32 once per
// half block.
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
constexpr uint32_t LUT_GRID_BYTES = 256 * 128, LUT_SIGN_BYTES = 128 * 128, LUT_BYTES = LUT_GRID_BYTES + LUT_SIGN_BYTES;

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

// The same with a zero accumulator on input (no registers to clear).
__device__ __forceinline__ void mma_s8_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// One group of the dispatch: rows [first, first + count) of the expert-sorted pair list.
struct VGroup { uint32_t expert, first, count, pad; };

// Quantised activation rows in global memory (quantize_rows_kernel).
struct QuantRows {
    const int8_t *digits;              // [rows][2][K]
    const int8_t *negated;             // [rows][2][K]
    const int *sums;                   // [rows][K/32][2]
    const float *scale;                // [rows]
};

struct GroupedArgs {
    DevTensor w0, w1;                  // gate and up, or down (w1 unused)
    const VGroup *groups;              // device list; n_groups[0] entries
    const uint32_t *n_groups;
    const uint32_t *row_to_pair;       // nullptr: pair = row (shared expert)
    uint32_t k_div;                    // input row = pair / k_div
    QuantRows in;
    const uint8_t *lut;                // IQ2_XXS tables image, LUT_BYTES
    float *out;                        // [pairs][n_out]
    uint32_t *status;
};

template <uint32_t TYPE> struct Fmt;
template <> struct Fmt<T_Q4_K> {
    static constexpr uint32_t BLOCK_BYTES = 144;
    static constexpr bool NEEDS_LUT = false;
    __host__ __device__ static uint32_t pitch(uint32_t nb) {           // row pitch = 8 words mod 32: no bank conflicts
        uint32_t p = nb * 144;
        while ((p / 4) % 32 != 8) p += 16;
        return p;
    }
};
template <> struct Fmt<T_IQ2_XXS> {
    static constexpr uint32_t BLOCK_BYTES = 64;                          // payload; fp16 d kept apart
    static constexpr bool NEEDS_LUT = true;
    __host__ __device__ static uint32_t pitch(uint32_t nb) { return nb * 64; }   // rows are swizzled in the image
};

// Shared-memory plan (byte offsets), the same on host and device.
struct Plan {
    uint32_t bars, lut, bslot, bslot_bytes, xq, xneg, xsum, meta, partial, stages, stage_bytes, total;
    uint32_t n_stages, kp, pitch, unit_rows, matrices, dsec, per_matrix;
};
template <uint32_t TYPE, int MODE>
__host__ __device__ inline Plan make_plan(uint32_t k_storage) {
    Plan p;
    const uint32_t nb = k_storage / 256;
    p.unit_rows = MODE == 0 ? 32 : 256;                                 // two row tiles per warp and unit, so that the barriers and the
                                                                         // partial-sum exchange of a unit are paid half as often
    p.matrices = MODE == 0 ? 2 : 1;
    p.kp = k_storage + 32;
    p.pitch = Fmt<TYPE>::pitch(nb);
    uint32_t at = 0;
    p.bars = at; at += 512;
    p.lut = at; if (Fmt<TYPE>::NEEDS_LUT) at += LUT_BYTES;
    // one activation slot: digits [8][kp], chunk sums [TOK][K/32] int2, metadata
    uint32_t b = 0;
    p.xq = b; b += 8 * p.kp;
    p.xneg = b;
    p.xsum = b; b += TOK * (k_storage / 32) * 8;
    p.meta = b; b += 64;                                                 // [0..3] pair, [4] count, [8..11] float scale
    p.bslot_bytes = (b + 127) & ~127u;
    p.bslot = at; at += 2 * p.bslot_bytes;
    p.partial = at; at += 2 * CW * 128 * 4;                              // [parity][warp][128 floats]: two row tiles of 64 values per warp
    at = (at + 127) & ~127u;
    p.dsec = p.unit_rows * p.pitch;                                      // IQ2_XXS: fp16 d after the payload rows
    uint32_t per_matrix = p.unit_rows * p.pitch + (TYPE == T_IQ2_XXS ? ((p.unit_rows * nb * 2 + 15) & ~15u) : 0);
    p.per_matrix = (per_matrix + 127) & ~127u;
    p.stage_bytes = p.per_matrix * p.matrices;
    p.stages = at;
    const uint32_t budget = 220u * 1024u;
    uint32_t n = at < budget ? (budget - at) / p.stage_bytes : 0;
    p.n_stages = n > 8 ? 8 : n;
    p.total = at + p.n_stages * p.stage_bytes;
    return p;
}

// ------------------------------------------------------------------------------------
// Per-format consumption of one half block (128 columns = 4 chunks) for rows g and g+8.
// facc[0] += row g . x[token t], facc[1] += row g+8 . x[token t] (both still to be scaled by dx).
// `act` points at the activation slot in use.
// ------------------------------------------------------------------------------------
template <uint32_t TYPE> struct Consume;

template <> struct Consume<T_Q4_K> {
    __device__ static __forceinline__ void half_block(const uint8_t *stage, const Plan &p, const uint8_t *, const uint8_t *act,
                                                      uint32_t nb, uint32_t row0, uint32_t half, uint32_t g, uint32_t t, float (&facc)[2]) {
        const uint32_t b = half >> 1, hb = half & 1u;
        const uint8_t *r0 = stage + (row0 + g) * p.pitch + b * 144u, *r1 = r0 + 8 * p.pitch;
        const uint4 h0 = *reinterpret_cast<const uint4 *>(r0), h1 = *reinterpret_cast<const uint4 *>(r1);
        uint32_t sc0, mn0, sc1, mn1;
        if (hb == 0) { sc0 = h0.y & 0x3f3f3f3fu; mn0 = h0.z & 0x3f3f3f3fu; sc1 = h1.y & 0x3f3f3f3fu; mn1 = h1.z & 0x3f3f3f3fu; }
        else {
            sc0 = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u); mn0 = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u);
            sc1 = (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u); mn1 = ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u);
        }
        const uint8_t *xq = act + p.xq + g * p.kp + (half * 4u) * 32u + 8u * t;
        const int2 *xsum = reinterpret_cast<const int2 *>(act + p.xsum) + t * (nb * 8u) + half * 4u;
        int qacc[4] = {0, 0, 0, 0}, macc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {                                 // sub-block pair: low and high nibbles
            const uint2 q0 = *reinterpret_cast<const uint2 *>(r0 + 16 + (hb * 2 + cc) * 32 + 8 * t);
            const uint2 q1 = *reinterpret_cast<const uint2 *>(r1 + 16 + (hb * 2 + cc) * 32 + 8 * t);
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                const int j = cc * 2 + nib;                              // chunk within the half block
                const uint2 bq = *reinterpret_cast<const uint2 *>(xq + j * 32);
                int c[4];
                mma_s8_zero(c, (q0.x >> (4 * nib)) & 0x0f0f0f0fu, (q1.x >> (4 * nib)) & 0x0f0f0f0fu,
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
    __device__ static __forceinline__ void half_block(const uint8_t *stage, const Plan &p, const uint8_t *lut, const uint8_t *act,
                                                      uint32_t nb, uint32_t row0, uint32_t half, uint32_t g, uint32_t t, float (&facc)[2]) {
        const uint32_t b = half >> 1;
        // groups 4*half .. 4*half+3 of the row sit at ((4*half) ^ swizzle) + j: the swizzle only
        // touches bits 2-3 of the group index
        const uint8_t *r0 = stage + (row0 + g) * p.pitch + (((half * 4u) ^ iq2_swizzle(g, nb)) * 8u), *r1 = r0 + 8 * p.pitch;
        const uint8_t *grid = lut + (threadIdx.x & 15u) * 8u;            // 64-bit reads: 16 copies
        const uint8_t *sign = lut + LUT_GRID_BYTES + (threadIdx.x & 7u) * 16u;   // 128-bit reads: 8 copies
        const uint8_t *xq = act + p.xq + g * p.kp + (half * 4u) * 32u + 8u * t;
        const uint32_t pick = 0x4440u + t, shift_s = 7 * t;              // byte t of the index word; 7-bit sign field t
        int iacc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint2 g0 = *reinterpret_cast<const uint2 *>(r0 + 8 * j), g1 = *reinterpret_cast<const uint2 *>(r1 + 8 * j);
            const uint32_t i0 = __byte_perm(g0.x, 0u, pick), i1 = __byte_perm(g1.x, 0u, pick);
            const uint32_t s0 = (g0.y >> shift_s) & 127u, s1 = (g1.y >> shift_s) & 127u;
            const uint2 v0 = *reinterpret_cast<const uint2 *>(grid + i0 * 128u), v1 = *reinterpret_cast<const uint2 *>(grid + i1 * 128u);
            const uint4 m0 = *reinterpret_cast<const uint4 *>(sign + s0 * 128u), m1 = *reinterpret_cast<const uint4 *>(sign + s1 * 128u);
            const uint2 bq = *reinterpret_cast<const uint2 *>(xq + j * 32);
            int c[4];
            // m.x/m.y: 0xff where the weight is negative; m.z/m.w: 0x01 there.  Magnitudes are
            // never zero, so (v ^ 0xff) + 1 = -v stays inside its byte.
            mma_s8_zero(c, (v0.x ^ m0.x) + m0.z, (v1.x ^ m1.x) + m1.z, (v0.y ^ m0.y) + m0.w, (v1.y ^ m1.y) + m1.w, bq.x, bq.y);
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

// Producer: stage one unit (unit_rows rows of each matrix).
template <uint32_t TYPE>
__device__ __forceinline__ void produce_unit(const GroupedArgs &a, const Plan &p, uint8_t *stage, uint64_t *full, uint32_t expert,
                                             uint32_t row0, uint32_t lane) {
    const uint32_t nb = a.w0.k_storage >> 8, rows = p.unit_rows;
    const uint32_t row_bytes = nb * Fmt<TYPE>::BLOCK_BYTES;
    const bool contiguous = p.pitch == row_bytes;
    if (lane == 0) mbar_expect_tx(full, p.matrices * (rows * row_bytes + (TYPE == T_IQ2_XXS ? rows * nb * 2 : 0)));
    __syncwarp();
    for (uint32_t m = 0; m < p.matrices; m++) {
        const DevTensor &w = m == 0 ? a.w0 : a.w1;
        const uint8_t *mat = w.data + (uint64_t)expert * w.expert_bytes;
        uint8_t *dst = stage + m * p.per_matrix;
        if (contiguous) {
            if (lane == 0) bulk_copy(dst, mat + (uint64_t)row0 * row_bytes, rows * row_bytes, full);
        } else {
            for (uint32_t r = lane; r < rows; r += 32) bulk_copy(dst + r * p.pitch, mat + (uint64_t)(row0 + r) * row_bytes, row_bytes, full);
        }
        if (TYPE == T_IQ2_XXS && lane == 1)
            bulk_copy(dst + p.dsec, mat + (uint64_t)w.n_out * nb * 64u + (uint64_t)row0 * nb * 2u, rows * nb * 2, full);
    }
}

// Producer: stage one group's activation digits, chunk sums and metadata.
template <uint32_t TYPE>
__device__ __forceinline__ void produce_group(const GroupedArgs &a, const Plan &p, uint8_t *slot, uint64_t *full, const VGroup grp,
                                              uint32_t lane) {
    const uint32_t K = a.w0.k_storage, sums_bytes = (K >> 5) * 8;
    const uint32_t per_token = 2 * K + sums_bytes;
    uint32_t row = 0;
    if (lane < grp.count) {
        const uint32_t pair = a.row_to_pair ? a.row_to_pair[grp.first + lane] : grp.first + lane;
        row = pair / a.k_div;
        reinterpret_cast<uint32_t *>(slot + p.meta)[lane] = pair;
        reinterpret_cast<float *>(slot + p.meta)[8 + lane] = a.in.scale[row];
    }
    if (lane == 4) reinterpret_cast<uint32_t *>(slot + p.meta)[4] = grp.count;
    __syncwarp();
    if (lane == 0) mbar_expect_tx(full, grp.count * per_token);
    __syncwarp();
    for (uint32_t tok = 0; tok < grp.count; tok++) {
        const uint32_t src_row = __shfl_sync(0xffffffffu, row, tok);
        if (lane < 2) bulk_copy(slot + p.xq + (2 * tok + lane) * p.kp, a.in.digits + ((uint64_t)src_row * 2 + lane) * K, K, full);
        else if (lane == 4) bulk_copy(slot + p.xsum + tok * sums_bytes, a.in.sums + (uint64_t)src_row * (K >> 5) * 2, sums_bytes, full);
    }
}

// MODE 0: gate + up + SwiGLU -> out = act.  MODE 1: down -> out (one row per pair).
template <uint32_t TYPE, int MODE>
__global__ void __launch_bounds__(NT, 1) grouped_mma_kernel(const GroupedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t K = a.w0.k_storage, nb = K >> 8, halves = K >> 7;
    const Plan p = make_plan<TYPE, MODE>(K);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + p.bars), *empty = full + 8, *bfull = full + 16, *bempty = full + 18, *lutbar = full + 20;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t n_groups = *a.n_groups;
    const uint32_t units_per_group = a.w0.n_out / p.unit_rows;
    const uint64_t total = (uint64_t)n_groups * units_per_group;
    const uint32_t u_begin = (uint32_t)(total * blockIdx.x / gridDim.x), u_end = (uint32_t)(total * (blockIdx.x + 1) / gridDim.x);
    if (u_begin == u_end) return;

    if (tid == 0) {
        for (uint32_t s = 0; s < p.n_stages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
        for (uint32_t s = 0; s < 2; s++) { mbar_init(&bfull[s], 1); mbar_init(&bempty[s], CW); }
        mbar_init(lutbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CW) {                                                    // ---- producer warp ----
        if (Fmt<TYPE>::NEEDS_LUT && lane == 0) {
            mbar_expect_tx(lutbar, LUT_BYTES);
            bulk_copy(smem + p.lut, a.lut, LUT_BYTES, lutbar);
        }
        uint32_t stage = 0, phase = 0, bslot = 0, bphase = 0, staged = 0, current = 0xffffffffu;
        bool alive = true;
        for (uint32_t u = u_begin; u < u_end && alive; u++) {
            const uint32_t gi = u / units_per_group;
            const VGroup grp = a.groups[gi];
            if (gi != current) {                                         // next group's activations, one slot ahead
                if (lane == 0 && staged >= 2) alive = mbar_wait(&bempty[bslot], bphase ^ 1u, a.status);
                alive = __shfl_sync(0xffffffffu, alive, 0);
                if (!alive) break;
                produce_group<TYPE>(a, p, smem + p.bslot + bslot * p.bslot_bytes, &bfull[bslot], grp, lane);
                staged++;
                if (++bslot == 2) { bslot = 0; bphase ^= 1u; }
                current = gi;
            }
            if (lane == 0 && u - u_begin >= p.n_stages) alive = mbar_wait(&empty[stage], phase ^ 1u, a.status);
            alive = __shfl_sync(0xffffffffu, alive, 0);
            if (!alive) break;
            produce_unit<TYPE>(a, p, smem + p.stages + stage * p.stage_bytes, &full[stage], grp.expert,
                               (u % units_per_group) * p.unit_rows, lane);
            if (++stage == p.n_stages) { stage = 0; phase ^= 1u; }
        }
        return;
    }

    // ---- consumer warps ----
    const uint32_t g = lane >> 2, t = lane & 3u;
    float *partial = reinterpret_cast<float *>(smem + p.partial);
    uint32_t stage = 0, phase = 0, parity = 0, current = 0xffffffffu, bslot = 1, bphase = 1;
    bool alive = true;
    if (Fmt<TYPE>::NEEDS_LUT) {
        if (lane == 0) alive = mbar_wait(lutbar, 0, a.status);
        alive = __shfl_sync(0xffffffffu, alive, 0);
    }
    const uint8_t *act = smem + p.bslot;
    for (uint32_t u = u_begin; u < u_end; u++) {
        const uint32_t gi = u / units_per_group, row_tile = (u % units_per_group) * p.unit_rows;
        if (gi != current) {                                             // switch to the next activation slot
            if (current != 0xffffffffu) {
                consumer_sync();                                         // epilogues of the old group have read its metadata
                if (lane == 0) mbar_arrive(&bempty[bslot]);
            }
            if (++bslot == 2) { bslot = 0; bphase ^= 1u; }
            if (alive && lane == 0) alive = mbar_wait(&bfull[bslot], bphase, a.status);
            alive = __shfl_sync(0xffffffffu, alive, 0);
            act = smem + p.bslot + bslot * p.bslot_bytes;
            current = gi;
        }
        if (alive && lane == 0) alive = mbar_wait(&full[stage], phase, a.status);
        alive = __shfl_sync(0xffffffffu, alive, 0);
        const uint8_t *st = smem + p.stages + stage * p.stage_bytes;
        float facc[2] = {0.0f, 0.0f}, facc2[2] = {0.0f, 0.0f};
        if (MODE == 0) {                                                 // warp = (matrix, k-slice of 8), both row tiles of the unit
            const uint32_t m = warp & 1u, ks = warp >> 1;
            if (alive)
                for (uint32_t h = ks; h < halves; h += 8) {
                    Consume<TYPE>::half_block(st + m * p.per_matrix, p, smem + p.lut, act, nb, 0, h, g, t, facc);
                    Consume<TYPE>::half_block(st + m * p.per_matrix, p, smem + p.lut, act, nb, 16, h, g, t, facc2);
                }
        } else {                                                         // warp = (row tile of 8, k-slice of 2)
            const uint32_t rt = warp & 7u, ks = warp >> 3;
            if (alive)
                for (uint32_t h = ks; h < halves; h += 2) {
                    Consume<TYPE>::half_block(st, p, smem + p.lut, act, nb, rt * 16, h, g, t, facc);
                    Consume<TYPE>::half_block(st, p, smem + p.lut, act, nb, 128 + rt * 16, h, g, t, facc2);
                }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
        if (++stage == p.n_stages) { stage = 0; phase ^= 1u; }
        float *mine = partial + (parity * CW + warp) * 128;
        mine[lane] = facc[0];                                            // (row g, token t) at 4g + t
        mine[32 + lane] = facc[1];                                       // (row g + 8, token t)
        mine[64 + lane] = facc2[0]; mine[96 + lane] = facc2[1];          // the second row tile: rows 16 + g, 24 + g (gate/up) or 128 + ... (down)
        consumer_sync();
        const float *part = partial + parity * CW * 128;
        const uint32_t *meta = reinterpret_cast<const uint32_t *>(act + p.meta);
        const float *tokscale = reinterpret_cast<const float *>(act + p.meta) + 8;
        const uint32_t count = meta[4];
        if (MODE == 0) {
            if (tid < 128) {                                             // 32 rows x 4 tokens
                const uint32_t row = tid >> 2, tok = tid & 3u;
                float gsum = 0.0f, usum = 0.0f;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) { gsum += part[(2 * ks) * 128 + tid]; usum += part[(2 * ks + 1) * 128 + tid]; }
                if (tok < count) {
                    const float dx = tokscale[tok];
                    gsum *= dx; usum *= dx;
                    const float e = __expf(-fabsf(gsum));
                    const float sig = gsum >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
                    const float v = gsum * sig * usum;
                    if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.out[(uint64_t)meta[tok] * a.w0.n_out + row_tile + row] = v;
                }
            }
        } else {                                                         // 256 rows x 4 tokens: two per consumer thread
            const uint32_t rt = tid >> 6, within = tid & 63u, tok = within & 3u;
            if (tok < count) {
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const float sum = (part[rt * 128 + half * 64 + within] + part[(8 + rt) * 128 + half * 64 + within]) * tokscale[tok];
                    if ((__float_as_uint(sum) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.out[(uint64_t)meta[tok] * a.w0.n_out + row_tile + half * 128 + rt * 16 + (within >> 2)] = sum;
                }
            }
        }
        parity ^= 1u;
    }
    if (current != 0xffffffffu) { consumer_sync(); if (lane == 0) mbar_arrive(&bempty[bslot]); }
}

// Two int8 digits per activation: x ~ dx * (q1 + q2 / 254), dx = max|x| / 127 per row.
// One CTA per row.  Also writes the negated digits (IQ2_XXS sign correction) and the per-chunk
// digit sums (Q4_K min term).  k is a multiple of 32.
// One CTA of 128 threads per row, float4 items: the row maximum first, then two int8 digits per value by the
// 1.5 * 2^23 rounding trick (the low byte of the rounded float's bit pattern is the digit), four digits packed
// with byte permutes, chunk sums by dp4a and three shuffles (eight consecutive lanes hold one 32-column chunk;
// both sums travel in one register, the second in the high half).  k % 32 == 0.
// row_list (optional): CTA b handles row row_list[*row_begin + b] (row_begin null: 0), and only while that index is
// below *row_end (the rows an expert-parallel rank's experts actually received, out of a launch sized for the most
// there can be).
__global__ void __launch_bounds__(128) quantize_rows_kernel(const float *__restrict__ x, uint32_t pitch, uint32_t k, int8_t *__restrict__ xq,
                                                            int8_t *__restrict__ xneg, int *__restrict__ xsum, float *__restrict__ xscale,
                                                            const uint32_t *__restrict__ row_list, const uint32_t *__restrict__ row_begin,
                                                            const uint32_t *__restrict__ row_end) {
    __shared__ float red[4];
    const uint32_t listed = row_list ? (row_begin ? *row_begin : 0u) + blockIdx.x : 0u;
    if (row_list && listed >= *row_end) return;
    const uint32_t row = row_list ? row_list[listed] : blockIdx.x;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, items = k >> 2;
    const float4 *src = reinterpret_cast<const float4 *>(x + (uint64_t)row * pitch);
    float amax = 0.0f;
    for (uint32_t i = tid; i < items; i += 128) {
        const float4 v = src[i];
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const bool usable = amax > 0.0f && amax <= 3.0e38f;
    const float dx = usable ? amax / 127.0f : 1.0f, inv = 1.0f / dx, inv2 = 254.0f / dx, magic = 12582912.0f;
    if (tid == 0) xscale[row] = usable ? dx : 0.0f;
    uint32_t *q1 = reinterpret_cast<uint32_t *>(xq + ((uint64_t)row * 2) * k), *q2 = reinterpret_cast<uint32_t *>(xq + ((uint64_t)row * 2 + 1) * k);
    uint32_t *n1 = reinterpret_cast<uint32_t *>(xneg + ((uint64_t)row * 2) * k), *n2 = reinterpret_cast<uint32_t *>(xneg + ((uint64_t)row * 2 + 1) * k);
    for (uint32_t i0 = 0; i0 < items; i0 += 128) {                      // items is a multiple of 8: whole groups of eight lanes
        const uint32_t i = i0 + tid;
        const bool live = i < items;
        const float4 v4 = live ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
        uint32_t ra[4], rb[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float v = usable ? vv[j] : 0.0f;
            const float r1 = fmaf(v, inv, magic), d1 = r1 - magic;
            const float r2 = fmaxf(-127.0f, fminf(127.0f, fmaf(-d1, dx, v) * inv2)) + magic;
            ra[j] = __float_as_uint(r1); rb[j] = __float_as_uint(r2);
        }
        const uint32_t hi = __byte_perm(__byte_perm(ra[0], ra[1], 0x0040), __byte_perm(ra[2], ra[3], 0x0040), 0x5410);
        const uint32_t lo = __byte_perm(__byte_perm(rb[0], rb[1], 0x0040), __byte_perm(rb[2], rb[3], 0x0040), 0x5410);
        if (live) {
            q1[i] = hi; q2[i] = lo;
            n1[i] = __vneg4(hi); n2[i] = __vneg4(lo);
        }
        int s = __dp4a((int)hi, 0x01010101, 0) + (__dp4a((int)lo, 0x01010101, 0) << 16);
        for (int o = 1; o < 8; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (live && (lane & 7u) == 0) {
            const int s1 = (int)(short)(s & 0xffff);
            reinterpret_cast<int2 *>(xsum)[(uint64_t)row * (k >> 5) + (i >> 3)] = make_int2(s1, (s - s1) >> 16);
        }
    }
}

// IQ2_XXS tables as the kernels want them in shared memory.  256 codebook vectors of 8 bytes,
// each 16 times (8 bytes apart, 128 bytes per entry): lane L reads copy L % 16 with a 64-bit
// load.  128 sign words of 16 bytes {mask lo, mask hi, ones lo, ones hi}, each 8 times (128
// bytes per entry): lane L reads copy L % 8 with a 128-bit load.  Neither has bank conflicts.
__global__ void build_lut_kernel(uint8_t *lut) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < 256 * 16 + 128 * 8; i += gridDim.x * blockDim.x) {
        if (i < 256 * 16) {
            const uint32_t entry = i >> 4, levels = c_iq2_levels[entry];
            uint32_t lo = 0, hi = 0;
            for (int j = 0; j < 4; j++) {
                lo |= iq2_magnitude((levels >> (2 * j)) & 3u) << (8 * j);
                hi |= iq2_magnitude((levels >> (2 * j + 8)) & 3u) << (8 * j);
            }
            *reinterpret_cast<uint2 *>(lut + entry * 128u + (i & 15u) * 8u) = make_uint2(lo, hi);
        } else {
            const uint32_t k = i - 256 * 16, entry = k >> 3, signs = iq2_signs8(entry);
            uint32_t lo = 0, hi = 0;
            for (int j = 0; j < 4; j++) {
                if ((signs >> j) & 1u) lo |= 0xffu << (8 * j);
                if ((signs >> (j + 4)) & 1u) hi |= 0xffu << (8 * j);
            }
            *reinterpret_cast<uint4 *>(lut + LUT_GRID_BYTES + entry * 128u + (k & 7u) * 16u) =
                make_uint4(lo, hi, lo & 0x01010101u, hi & 0x01010101u);
        }
    }
}

// y[t, c] = sum over slots in slot order of weight[t, s] * out[t*k + s, c] + sigmoid(slogit[t]) * shared_out[t, c]
// (picoforge src/qwen4_moe.c:362-380).
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ out, const float *__restrict__ shared_out,
                                                      const float *__restrict__ weights, const float *__restrict__ shared_logit,
                                                      uint32_t k, uint32_t hidden, float *__restrict__ y, float *__restrict__ routed,
                                                      uint32_t *status, HcAdd hc) {
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
    if (!hc_add(hc, t, c, hidden, total)) atomicOr(status, QW4SH_ERR_NONFINITE);
}

// Groups of at most four rows out of the expert-sorted lists.
// One CTA, thread i owns active expert i (then i + 1024, ...); a block-wide exclusive scan of the group counts gives
// every expert its place in the list: active experts in ascending order, each expert's groups by ascending row.
__global__ void __launch_bounds__(1024) build_groups_kernel(const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ active,
                                                            VGroup *groups, uint32_t *n_groups) {
    __shared__ uint32_t wsum[32];
    __shared__ uint32_t s_base;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, n_active = active[0];
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (uint32_t i0 = 0; i0 < n_active; i0 += 1024) {
        const uint32_t i = i0 + tid;
        uint32_t e = 0, first = 0, end = 0;
        if (i < n_active) { e = active[1 + i]; first = offsets[e]; end = offsets[e + 1]; }
        const uint32_t count = (end - first + TOK - 1) / TOK;
        uint32_t scan = count;
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
        uint32_t at = s_base + wsum[warp] + scan - count;
        for (uint32_t r = first; r < end; r += TOK) groups[at++] = VGroup{e, r, min((uint32_t)TOK, end - r), 0};
        __syncthreads();
        if (tid == 1023) s_base = at;                                // end of the last thread = end of this pass
        __syncthreads();
    }
    if (tid == 0) *n_groups = s_base;
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

static uint8_t *g_lut[64] = {nullptr};
static const uint8_t *lut_image() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (!g_lut[device]) {
        uint8_t *p = nullptr;
        if (cudaMalloc(&p, LUT_BYTES) != cudaSuccess) return nullptr;
        build_lut_kernel<<<24, 256>>>(p);
        if (qw4sh_note_launch("build_lut_kernel") || cudaDeviceSynchronize() != cudaSuccess) { cudaFree(p); return nullptr; }
        g_lut[device] = p;
    }
    return g_lut[device];
}

extern "C" int qw4sh_mma_supported(const QW4ShTensor *w, int mode) {
    if (w->type != T_Q4_K && w->type != T_IQ2_XXS) return 0;
    if (w->k_storage % 256 || w->k_storage > KMAX || w->k_logical != w->k_storage) return 0;
    if (w->n_out % (mode == 0 ? 32 : 256)) return 0;
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
// Input rows are the quantised rows of quantize_rows (row = pair / k_div).
extern "C" int qw4sh_grouped_mma(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                                 const uint32_t *row_to_pair, uint32_t k_div, const int8_t *digits, const int8_t *negated,
                                 const int *sums, const float *scale, float *out, uint32_t *status, int ctas, void *stream) {
    GroupedArgs a;
    a.w0 = dev(*w0); a.w1 = dev(w1 ? *w1 : *w0);
    a.groups = (const VGroup *)groups; a.n_groups = n_groups; a.row_to_pair = row_to_pair; a.k_div = k_div;
    a.in.digits = digits; a.in.negated = negated; a.in.sums = sums; a.in.scale = scale;
    a.lut = nullptr; a.out = out; a.status = status;
    if (w0->type == T_IQ2_XXS && !(a.lut = lut_image())) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (w0->type == T_Q4_K) return mode == 0 ? launch_grouped<T_Q4_K, 0>(a, ctas, s) : launch_grouped<T_Q4_K, 1>(a, ctas, s);
    return mode == 0 ? launch_grouped<T_IQ2_XXS, 0>(a, ctas, s) : launch_grouped<T_IQ2_XXS, 1>(a, ctas, s);
}

extern "C" int qw4sh_prepare_mma(void) { return lut_image() ? 0 : -1; }
extern "C" const uint8_t *qw4sh_lut_image(void) { return lut_image(); }

// Rows of k floats, `pitch` floats apart.
extern "C" int qw4sh_quantize_rows_pitched(const float *x, uint32_t pitch, uint32_t rows, uint32_t k, int8_t *xq, int8_t *xneg, int *xsum,
                                           float *xscale, void *stream) {
    if (!rows) return 0;
    quantize_rows_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(x, pitch, k, xq, xneg, xsum, xscale, nullptr, nullptr, nullptr);
    return qw4sh_note_launch("quantize_rows_kernel");
}
extern "C" int qw4sh_quantize_rows_listed(const float *x, uint32_t pitch, uint32_t max_rows, uint32_t k, const uint32_t *row_list,
                                          const uint32_t *row_begin, const uint32_t *row_end, int8_t *xq, int8_t *xneg, int *xsum, float *xscale,
                                          void *stream) {
    if (!max_rows) return 0;
    quantize_rows_kernel<<<max_rows, 128, 0, (cudaStream_t)stream>>>(x, pitch, k, xq, xneg, xsum, xscale, row_list, row_begin, row_end);
    return qw4sh_note_launch("quantize_rows_kernel");
}
extern "C" int qw4sh_quantize_rows(const float *x, uint32_t rows, uint32_t k, int8_t *xq, int8_t *xneg, int *xsum, float *xscale, void *stream) {
    return qw4sh_quantize_rows_pitched(x, k, rows, k, xq, xneg, xsum, xscale, stream);
}
extern "C" int qw4sh_combine(const float *out, const float *shared_out, const float *weights, const float *shared_logit, uint32_t k,
                             uint32_t hidden, uint32_t tokens, float *y, float *routed, uint32_t *status, float *hc_residual,
                             const float *hc_inject, uint32_t hc_streams, void *stream) {
    const HcAdd hc = {hc_residual, hc_inject, hc_streams};
    combine_kernel<<<dim3((hidden + 255) / 256, tokens), 256, 0, (cudaStream_t)stream>>>(out, shared_out, weights, shared_logit, k, hidden, y, routed, status, hc);
    return qw4sh_note_launch("combine_kernel");
}
extern "C" int qw4sh_build_groups(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream) {
    build_groups_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(offsets, active, (VGroup *)groups, n_groups);
    return qw4sh_note_launch("build_groups_kernel");
}
extern "C" int qw4sh_build_dense_groups(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream) {
    build_dense_groups_kernel<<<(tokens / TOK + 256) / 256, 256, 0, (cudaStream_t)stream>>>(tokens, (VGroup *)groups, n_groups);
    return qw4sh_note_launch("build_dense_groups_kernel");
}
