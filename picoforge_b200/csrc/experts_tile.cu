// Expert products for groups of up to 16 token rows of one expert on the int8 tensor-core path, with each
// weight fragment built ONCE and applied to all of the group's 4-token column tiles.
//
// Between the one-kernel decode path (<= 4 tokens) and the tcgen05 grouped GEMM (dense groups) lies the regime of
// batched decode and sparse prefill: an expert sees a handful to a few dozen rows.  A tcgen05.mma costs the same
// 144 cycles whatever its N, so few rows waste it; here the cost per weight is the fragment build plus about a
// dozen instructions per column tile.
//
// A CTA takes one group at a time: the two-int8-digit images of the group's activation rows (quantize_rows) come
// into shared memory once, by one bulk copy per digit row, and every warp then walks row tiles of the expert:
// gate/up tiles are 8 gate rows + the same 8 up rows (MMA rows 0-7 and 8-15, so SwiGLU stays in the lane), down
// tiles 16 rows.  A warp streams its tile's packed rows slice by slice with TMA bulk copies into its own
// two-stage ring and runs mma.sync.m16n8k32.s8 on the raw codes against the digits.  No cross-warp reduction; one
// CTA barrier per group.  (Digits read straight from global memory, the first form of this kernel, left every
// chunk step waiting for an L2 round trip.)
//
// Every mbarrier wait is bounded (about a second) and then records QW4SH_ERR_STATE.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "cuda_shim.h"
#include "formats.cuh"

namespace qw4 {

constexpr int TW = 12;                          // warps per CTA
constexpr int TT = TW * 32;
constexpr int TNS = 2;                          // ring stages per warp
constexpr int TNT = 4;                          // column tiles per group
constexpr uint32_t TROWS = 4 * TNT;             // token rows per group
constexpr uint32_t T_LUT_GRID = 256 * 128, T_LUT_SIGN = 128 * 128, T_LUT_BYTES = T_LUT_GRID + T_LUT_SIGN;
// bytes per ring stage: Q4_K 16 x 288; IQ2_XXS 4096 payload + up to 512 super-scales; Q2_K 4096 codes + 1024 scale bytes + 256
template <uint32_t TYPE> struct TStage { static constexpr uint32_t BYTES = TYPE == T_Q2_K ? 5376u : 4608u; };

struct TGroup { uint32_t expert, first, count, pad; };

struct TileArgs {
    DevTensor w0, w1;                           // gate and up, or down (w1 unused)
    const TGroup *groups;
    const uint32_t *n_groups;
    const uint32_t *row_to_pair;                // nullptr: pair = row (shared expert)
    uint32_t k_div;                             // input row = pair / k_div
    const int8_t *digits;                       // [rows][2][K]
    const int *sums;                            // [rows][K / 32][2] (not read: minima go through the tensor core)
    const float *scale;                         // [rows]
    const uint8_t *lut;                         // IQ2_XXS tables image
    float *out;                                 // gate/up: act [pairs][n_out]; down: out [pairs][n_out]
    uint32_t *status;
    uint32_t use_maps;                          // gate/up: the section maps passed beside this struct are valid
};
struct TileMaps { CUtensorMap m[2][3]; };       // [gate, up][section]

__device__ __forceinline__ uint32_t ts_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ts_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tbar_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ts_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(ts_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool tbar_wait(uint64_t *bar, uint32_t parity, uint32_t *status) {
    if (tbar_try(bar, parity)) return true;
    const long long start = clock64();
    while (!tbar_try(bar, parity)) {
        if (clock64() - start > (1ll << 31)) { atomicOr(status, QW4SH_ERR_STATE); return false; }
    }
    return true;
}
__device__ __forceinline__ void tbulk(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(ts_u32(dst_smem)), "l"(src), "r"(bytes), "r"(ts_u32(bar)) : "memory");
}
// Rows [y, y + 8) of expert z, 32-bit words [x, x + box) of each, through a 3-D tensor map {words of a row's
// section, rows of an expert, experts}: eight row pieces that lie a row apart in memory as ONE request.
__device__ __forceinline__ void ttma_rows(void *dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(ts_u32(dst_smem)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(ts_u32(bar)) : "memory");
}
__device__ __forceinline__ void tproxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmma_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void tmma_acc(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <uint32_t TYPE> struct TGeo;
template <> struct TGeo<T_Q4_K> { static constexpr uint32_t SLICE_BLOCKS = 2, BLOCK_BYTES = 144; };
template <> struct TGeo<T_IQ2_XXS> { static constexpr uint32_t SLICE_BLOCKS = 4, BLOCK_BYTES = 64; };
template <> struct TGeo<T_Q2_K> { static constexpr uint32_t SLICE_BLOCKS = 4, BLOCK_BYTES = 64; };       // codes; scale bytes and super-scales apart

// The two rows of a lane inside a ring stage: packed codes, and where the format keeps them apart its
// sub-block scale bytes (Q2_K) and super-scales (IQ2_XXS: fp16 d per block; Q2_K: {d, dmin} per block).
struct RowView {
    const uint8_t *r0, *r1, *aux0, *aux1, *dd0, *dd1;
    uint32_t swz;                                // IQ2_XXS: group swizzle of these rows
};

// One span of `halves` half blocks (128 columns each) of rows r0 / r1 against every column tile; the span starts at
// half block `first_half` of the row.  `bl` is the lane's place in the staged digits: digit row g (token g / 2 of
// a column tile, digit g & 1) at the lane's 8-column phase; column tile n is `tile_pitch` bytes further on.
// f[n][0] += row g . x[token 4n + t], f[n][1] += row g + 8 . x[token 4n + t] (in digit units).
template <uint32_t TYPE> struct TileHalves;

// Q4_K: the 4-bit codes are the A operand; the 6-bit sub-block minimum goes through a second MMA whose A operand
// is the minimum replicated over the lane's columns, so both sums come out of the tensor core.
template <> struct TileHalves<T_Q4_K> {
    static __device__ __forceinline__ void run(const RowView &v, uint32_t halves, uint32_t first_half, const uint8_t *, uint32_t t,
                                               const uint8_t *bl, uint32_t tile_pitch, uint32_t tiles, float (&f)[TNT][2]) {
        const uint8_t *r0 = v.r0, *r1 = v.r1;
        const float lo = 1.0f / 254.0f;
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++) {
            const uint8_t *b0 = r0 + (h >> 1) * 144u, *b1 = r1 + (h >> 1) * 144u;
            const uint32_t hb = h & 1u;
            const uint8_t *bh = bl + (first_half + h) * 128u;
            const uint4 h0 = *reinterpret_cast<const uint4 *>(b0), h1 = *reinterpret_cast<const uint4 *>(b1);
            uint32_t sc0, mn0, sc1, mn1;
            if (hb == 0) { sc0 = h0.y & 0x3f3f3f3fu; mn0 = h0.z & 0x3f3f3f3fu; sc1 = h1.y & 0x3f3f3f3fu; mn1 = h1.z & 0x3f3f3f3fu; }
            else {
                sc0 = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u); mn0 = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u);
                sc1 = (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u); mn1 = ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u);
            }
            const float d0 = __half2float(__ushort_as_half((uint16_t)(h0.x & 0xffffu))), n0 = __half2float(__ushort_as_half((uint16_t)(h0.x >> 16)));
            const float d1 = __half2float(__ushort_as_half((uint16_t)(h1.x & 0xffffu))), n1 = __half2float(__ushort_as_half((uint16_t)(h1.x >> 16)));
            // integer sums over the half block: codes x 6-bit scale by multiply-add, minima accumulated by the tensor core
            int iq[TNT][4], im[TNT][4];
#pragma unroll
            for (int n = 0; n < TNT; n++)
#pragma unroll
                for (int r = 0; r < 4; r++) { iq[n][r] = 0; im[n][r] = 0; }
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const uint2 q0 = *reinterpret_cast<const uint2 *>(b0 + 16 + (hb * 2 + cc) * 32 + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(b1 + 16 + (hb * 2 + cc) * 32 + 8 * t);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int j = cc * 2 + nib;
                    const uint32_t a0 = (q0.x >> (4 * nib)) & 0x0f0f0f0fu, a1 = (q1.x >> (4 * nib)) & 0x0f0f0f0fu;
                    const uint32_t a2 = (q0.y >> (4 * nib)) & 0x0f0f0f0fu, a3 = (q1.y >> (4 * nib)) & 0x0f0f0f0fu;
                    const int s0 = (int)((sc0 >> (8 * j)) & 0xffu), s1 = (int)((sc1 >> (8 * j)) & 0xffu);
                    const uint32_t m0 = ((mn0 >> (8 * j)) & 0xffu) * 0x01010101u, m1 = ((mn1 >> (8 * j)) & 0xffu) * 0x01010101u;
#pragma unroll
                    for (int n = 0; n < TNT; n++) {
                        if ((uint32_t)n < tiles) {
                            const uint2 bq = *reinterpret_cast<const uint2 *>(bh + n * tile_pitch + j * 32);
                            int c[4];
                            tmma_zero(c, a0, a1, a2, a3, bq.x, bq.y);
                            tmma_acc(im[n], m0, m1, m0, m1, bq.x, bq.y);
                            iq[n][0] += c[0] * s0; iq[n][1] += c[1] * s0; iq[n][2] += c[2] * s1; iq[n][3] += c[3] * s1;
                        }
                    }
                }
            }
#pragma unroll
            for (int n = 0; n < TNT; n++) {
                if ((uint32_t)n < tiles) {
                    f[n][0] += d0 * fmaf((float)iq[n][1], lo, (float)iq[n][0]) - n0 * fmaf((float)im[n][1], lo, (float)im[n][0]);
                    f[n][1] += d1 * fmaf((float)iq[n][3], lo, (float)iq[n][2]) - n1 * fmaf((float)im[n][3], lo, (float)im[n][2]);
                }
            }
        }
    }
};

template <> struct TileHalves<T_IQ2_XXS> {
    static __device__ __forceinline__ void run(const RowView &v, uint32_t halves, uint32_t first_half, const uint8_t *lut, uint32_t t,
                                               const uint8_t *bl, uint32_t tile_pitch, uint32_t tiles, float (&f)[TNT][2]) {
        const uint8_t *r0 = v.r0, *r1 = v.r1;
        const uint16_t *d0p = reinterpret_cast<const uint16_t *>(v.dd0), *d1p = reinterpret_cast<const uint16_t *>(v.dd1);
        const uint32_t swz = v.swz;
        const uint8_t *grid = lut + (threadIdx.x & 15u) * 8u;
        const uint8_t *sign = lut + T_LUT_GRID + (threadIdx.x & 7u) * 16u;
        const uint32_t pick = 0x4440u + t, shift_s = 7 * t;
        const float lo = 1.0f / 254.0f;
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++) {
            const uint32_t at = ((h * 4u) ^ swz) * 8u;
            const uint8_t *bh = bl + (first_half + h) * 128u;
            const float d0 = __half2float(__ushort_as_half(d0p[h >> 1])) * 0.125f, d1 = __half2float(__ushort_as_half(d1p[h >> 1])) * 0.125f;
            int iq[TNT][4];
#pragma unroll
            for (int n = 0; n < TNT; n++)
#pragma unroll
                for (int r = 0; r < 4; r++) iq[n][r] = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 g0 = *reinterpret_cast<const uint2 *>(r0 + at + 8 * j), g1 = *reinterpret_cast<const uint2 *>(r1 + at + 8 * j);
                const uint32_t i0 = __byte_perm(g0.x, 0u, pick), i1 = __byte_perm(g1.x, 0u, pick);
                const uint32_t s0 = (g0.y >> shift_s) & 127u, s1 = (g1.y >> shift_s) & 127u;
                const uint2 v0 = *reinterpret_cast<const uint2 *>(grid + i0 * 128u), v1 = *reinterpret_cast<const uint2 *>(grid + i1 * 128u);
                const uint4 m0 = *reinterpret_cast<const uint4 *>(sign + s0 * 128u), m1 = *reinterpret_cast<const uint4 *>(sign + s1 * 128u);
                const uint32_t a0 = (v0.x ^ m0.x) + m0.z, a1 = (v1.x ^ m1.x) + m1.z, a2 = (v0.y ^ m0.y) + m0.w, a3 = (v1.y ^ m1.y) + m1.w;
                const int w0 = (int)((g0.y >> 27) | 1u), w1 = (int)((g1.y >> 27) | 1u);         // 2 * scale + 1
#pragma unroll
                for (int n = 0; n < TNT; n++) {
                    if ((uint32_t)n < tiles) {
                        const uint2 bq = *reinterpret_cast<const uint2 *>(bh + n * tile_pitch + j * 32);
                        int c[4];
                        tmma_zero(c, a0, a1, a2, a3, bq.x, bq.y);
                        iq[n][0] += c[0] * w0; iq[n][1] += c[1] * w0; iq[n][2] += c[2] * w1; iq[n][3] += c[3] * w1;
                    }
                }
            }
#pragma unroll
            for (int n = 0; n < TNT; n++) {
                if ((uint32_t)n < tiles) {
                    f[n][0] += d0 * fmaf((float)iq[n][1], lo, (float)iq[n][0]);
                    f[n][1] += d1 * fmaf((float)iq[n][3], lo, (float)iq[n][2]);
                }
            }
        }
    }
};

// Q2_K in the resident image: 64 code bytes per block, 16 scale/min bytes per block, one word {d, dmin} per
// block, each in its own section.  A 32-column chunk spans two 16-column sub-blocks; lane (g, t) holds eight
// columns of ONE sub-block, so the 4-bit sub-block scale is multiplied into the 2-bit codes (<= 45, still int8) and
// the minimum goes through a second MMA whose A operand is the minimum replicated over the lane's columns: both
// sums come out of the tensor core, no per-16-column digit sums needed.
template <> struct TileHalves<T_Q2_K> {
    static __device__ __forceinline__ void run(const RowView &v, uint32_t halves, uint32_t first_half, const uint8_t *, uint32_t t,
                                               const uint8_t *bl, uint32_t tile_pitch, uint32_t tiles, float (&f)[TNT][2]) {
        const float lo = 1.0f / 254.0f;
        const uint8_t *r0 = v.r0, *r1 = v.r1, *s0 = v.aux0, *s1 = v.aux1;
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++) {
            const uint32_t blk = h >> 1, hb = h & 1u;
            const uint8_t *bh = bl + (first_half + h) * 128u;
            const uint2 q0 = *reinterpret_cast<const uint2 *>(r0 + blk * 64u + hb * 32u + 8u * t);
            const uint2 q1 = *reinterpret_cast<const uint2 *>(r1 + blk * 64u + hb * 32u + 8u * t);
            const uint2 w0 = *reinterpret_cast<const uint2 *>(s0 + blk * 16u + hb * 8u), w1 = *reinterpret_cast<const uint2 *>(s1 + blk * 16u + hb * 8u);
            const uint32_t dd0 = *reinterpret_cast<const uint32_t *>(v.dd0 + blk * 4u), dd1 = *reinterpret_cast<const uint32_t *>(v.dd1 + blk * 4u);
            const float d0 = __half2float(__ushort_as_half((uint16_t)(dd0 & 0xffffu))), n0 = __half2float(__ushort_as_half((uint16_t)(dd0 >> 16)));
            const float d1 = __half2float(__ushort_as_half((uint16_t)(dd1 & 0xffffu))), n1 = __half2float(__ushort_as_half((uint16_t)(dd1 >> 16)));
            int iq[TNT][4], im[TNT][4];                                         // both accumulated over the half block by the tensor core
#pragma unroll
            for (int n = 0; n < TNT; n++)
#pragma unroll
                for (int r = 0; r < 4; r++) { iq[n][r] = 0; im[n][r] = 0; }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t sh = 8u * ((j & 1) * 2 + (t >> 1));
                const uint32_t b0 = ((j < 2 ? w0.x : w0.y) >> sh) & 0xffu, b1 = ((j < 2 ? w1.x : w1.y) >> sh) & 0xffu;
                const uint32_t sc0 = b0 & 15u, sc1 = b1 & 15u, m0 = (b0 >> 4) * 0x01010101u, m1 = (b1 >> 4) * 0x01010101u;
                const uint32_t a0 = ((q0.x >> (2 * j)) & 0x03030303u) * sc0, a1 = ((q1.x >> (2 * j)) & 0x03030303u) * sc1;
                const uint32_t a2 = ((q0.y >> (2 * j)) & 0x03030303u) * sc0, a3 = ((q1.y >> (2 * j)) & 0x03030303u) * sc1;
#pragma unroll
                for (int n = 0; n < TNT; n++) {
                    if ((uint32_t)n < tiles) {
                        const uint2 bq = *reinterpret_cast<const uint2 *>(bh + n * tile_pitch + j * 32);
                        tmma_acc(iq[n], a0, a1, a2, a3, bq.x, bq.y);
                        tmma_acc(im[n], m0, m1, m0, m1, bq.x, bq.y);
                    }
                }
            }
#pragma unroll
            for (int n = 0; n < TNT; n++) {
                if ((uint32_t)n < tiles) {
                    f[n][0] += d0 * fmaf((float)iq[n][1], lo, (float)iq[n][0]) - n0 * fmaf((float)im[n][1], lo, (float)im[n][0]);
                    f[n][1] += d1 * fmaf((float)iq[n][3], lo, (float)iq[n][2]) - n1 * fmaf((float)im[n][3], lo, (float)im[n][2]);
                }
            }
        }
    }
};

// Shared-memory plan: barriers | tables (IQ2_XXS) | digits [2 * TROWS rows][K + 32] | rings.
__host__ __device__ inline uint32_t tile_digit_pitch(uint32_t k) { return k + 32; }     // 8 words mod 32: the lanes' 64-bit reads miss each other's banks
template <uint32_t TYPE>
__host__ __device__ inline uint32_t tile_smem_bytes(uint32_t k) {
    return 512 + (TYPE == T_IQ2_XXS ? T_LUT_BYTES : 0) + 2 * TROWS * tile_digit_pitch(k) + TW * TNS * TStage<TYPE>::BYTES;
}

// MODE 0: gate + up + SwiGLU -> act; MODE 1: down -> out.
template <uint32_t TYPE, int MODE>
__global__ void __launch_bounds__(TT, 1) expert_tile_kernel(const TileArgs a, const __grid_constant__ TileMaps maps) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool LUT = TYPE == T_IQ2_XXS;
    constexpr uint32_t SB = TGeo<TYPE>::SLICE_BLOCKS, BB = TGeo<TYPE>::BLOCK_BYTES, STAGE = TStage<TYPE>::BYTES;
    uint64_t *ringbar = reinterpret_cast<uint64_t *>(smem);                    // [TW][TNS], then the table barrier, then the digits barrier
    uint64_t *lutbar = ringbar + TW * TNS, *digitbar = lutbar + 1;
    const uint8_t *lut = smem + 512;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t K = a.w0.k_storage, nb = K >> 8, n_out = a.w0.n_out, kp = tile_digit_pitch(K);
    uint8_t *digits_s = smem + 512 + (LUT ? T_LUT_BYTES : 0);
    uint8_t *ring = digits_s + 2 * TROWS * kp + warp * TNS * STAGE;
    uint64_t *bar = ringbar + warp * TNS;
    const uint32_t tile_rows = MODE == 0 ? 8u : 16u, tiles = n_out / tile_rows;
    const uint32_t row_bytes = nb * BB;                                        // Q4_K, IQ2_XXS payload (Q2_K: code bytes)
    // MODE 0 streams K in slices; MODE 1 fetches a whole 16-row tile (K <= 512 for Q4_K, <= 1024 otherwise)
    const uint32_t spu = MODE == 0 ? nb / SB : 1u;
    if (tid == 0) {
        for (uint32_t i = 0; i < TW * TNS; i++) tbar_init(&ringbar[i], 1);
        tbar_init(lutbar, 1);
        tbar_init(digitbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (LUT && tid == 0) {
        tbar_expect(lutbar, T_LUT_BYTES);
        tbulk(smem + 512, a.lut, T_LUT_BYTES, lutbar);
    }
    const uint32_t n_groups = *a.n_groups;
    bool alive = true;
    if (LUT) alive = tbar_wait(lutbar, 0, a.status);                           // also without work: no copy may be in flight when the CTA leaves
    const uint8_t *bl = digits_s + g * kp + 8 * t;                              // digit row g of a column tile, this lane's column phase
    // A work item is (group, part): with few groups each group's row tiles are dealt to `parts` CTAs, one pass of TW
    // tiles at a time (every CTA of a group stages the group's digits for itself); with many groups a CTA takes whole
    // groups and stages the digits once for all of the expert's tiles.
    const uint32_t rounds = (tiles + TW - 1) / TW;
    const uint32_t parts = n_groups < 2 * gridDim.x ? rounds : 1u;             // restaging the digits costs a few percent of a pass
    uint32_t ring_base = 0;                                                     // slices this warp has pushed through its ring
    uint32_t turn = 0;                                                          // items this CTA has taken: parity of the digits barrier
#pragma unroll 1
    for (uint32_t item = blockIdx.x; item < n_groups * parts; item += gridDim.x, turn++) {
        const uint32_t gi = item / parts, part = item % parts;
        const uint32_t tile0 = warp + TW * part, tile_step = TW * parts;       // this warp's row tiles: tile0, tile0 + tile_step, ...
        const uint32_t mine = tiles > tile0 ? (tiles - 1 - tile0) / tile_step + 1 : 0;
        const TGroup grp = a.groups[gi];
        const uint32_t count = min(grp.count, TROWS), n_tiles = (count + 3) >> 2;
        if (grp.count > TROWS && tid == 0) atomicOr(a.status, QW4SH_ERR_STATE);   // a list built for another kernel
        // this lane's token of the group: pair, input row
        uint32_t my_pair = 0;
        if (lane < count) my_pair = a.row_to_pair ? a.row_to_pair[grp.first + lane] : grp.first + lane;
        const uint32_t my_row = my_pair / a.k_div;
        __syncthreads();                                                        // every warp is done with the previous group's digits
        if (warp == 0 && alive) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (lane == 0) tbar_expect(digitbar, count * 2 * K);
            __syncwarp();
            if (lane < count) {
                const int8_t *src = a.digits + (uint64_t)my_row * 2 * K;
                tbulk(digits_s + (2 * lane) * kp, src, K, digitbar);
                tbulk(digits_s + (2 * lane + 1) * kp, src + K, K, digitbar);
            }
        }
        auto issue = [&](uint32_t n) {                                         // slice n of this warp's tiles of this group
            const uint32_t row0 = (tile0 + (n / spu) * tile_step) * tile_rows, s = n % spu, at = ring_base + n;
            uint8_t *stage = ring + (at % TNS) * STAGE;
            uint64_t *full = &bar[at % TNS];
            if (TYPE == T_Q2_K) {
                // three sections per matrix: codes, scale bytes, {d, dmin}; in the stage at 0, 4096 and 5120
                const uint64_t blocks = (uint64_t)n_out * nb;
                if (MODE == 0 && a.use_maps) {
                    if (lane == 0) tbar_expect(full, 16 * (SB * 84u));
                    __syncwarp();
                    if (lane < 6) {                                             // lane = 3 * matrix + section
                        const uint32_t mx = lane / 3, sec = lane % 3;
                        const uint32_t piece = sec == 0 ? SB * 64u : sec == 1 ? SB * 16u : SB * 4u, base = sec == 0 ? 0u : sec == 1 ? 4096u : 5120u;
                        ttma_rows(stage + base + mx * 8 * piece, &maps.m[mx][sec], s * (piece / 4), row0, grp.expert, full);
                    }
                } else if (MODE == 0) {
                    if (lane == 0) tbar_expect(full, 16 * (SB * 84u));
                    __syncwarp();
                    if (lane < 16) {
                        const DevTensor &w = lane < 8 ? a.w0 : a.w1;
                        const uint8_t *mat = w.data + (uint64_t)grp.expert * w.expert_bytes;
                        const uint64_t b0 = (uint64_t)(row0 + (lane & 7u)) * nb + s * SB;
                        tbulk(stage + lane * (SB * 64u), mat + b0 * 64u, SB * 64u, full);
                        tbulk(stage + 4096 + lane * (SB * 16u), mat + blocks * 64u + b0 * 16u, SB * 16u, full);
                        tbulk(stage + 5120 + lane * (SB * 4u), mat + blocks * 80u + b0 * 4u, SB * 4u, full);
                    }
                } else if (lane == 0) {
                    const uint8_t *mat = a.w0.data + (uint64_t)grp.expert * a.w0.expert_bytes;
                    const uint64_t b0 = (uint64_t)row0 * nb;
                    tbar_expect(full, 16 * nb * 84u);
                    tbulk(stage, mat + b0 * 64u, 16 * nb * 64u, full);
                    tbulk(stage + 4096, mat + blocks * 64u + b0 * 16u, 16 * nb * 16u, full);
                    tbulk(stage + 5120, mat + blocks * 80u + b0 * 4u, 16 * nb * 4u, full);
                }
            } else if (MODE == 0 && a.use_maps) {
                constexpr uint32_t slice_bytes = SB * BB;
                if (lane == 0) tbar_expect(full, 16 * slice_bytes + (LUT ? 2 * 8 * nb * 2 : 0));
                __syncwarp();
                if (lane < 2) ttma_rows(stage + lane * 8 * slice_bytes, &maps.m[lane][0], s * (slice_bytes / 4), row0, grp.expert, full);
                else if (LUT && lane < 4) {
                    const DevTensor &w = lane == 2 ? a.w0 : a.w1;
                    const uint8_t *mat = w.data + (uint64_t)grp.expert * w.expert_bytes;
                    tbulk(stage + 16 * slice_bytes + (lane - 2) * 8 * nb * 2, mat + (uint64_t)n_out * nb * 64u + (uint64_t)row0 * nb * 2u, 8 * nb * 2, full);
                }
            } else if (MODE == 0) {
                constexpr uint32_t slice_bytes = SB * BB;
                if (lane == 0) tbar_expect(full, 16 * slice_bytes + (LUT ? 2 * 8 * nb * 2 : 0));
                __syncwarp();
                if (lane < 16) {
                    const DevTensor &w = lane < 8 ? a.w0 : a.w1;
                    const uint8_t *mat = w.data + (uint64_t)grp.expert * w.expert_bytes;
                    tbulk(stage + lane * slice_bytes, mat + (uint64_t)(row0 + (lane & 7u)) * row_bytes + s * slice_bytes, slice_bytes, full);
                } else if (LUT && lane < 18) {
                    const DevTensor &w = lane == 16 ? a.w0 : a.w1;
                    const uint8_t *mat = w.data + (uint64_t)grp.expert * w.expert_bytes;
                    tbulk(stage + 16 * slice_bytes + (lane - 16) * 8 * nb * 2, mat + (uint64_t)n_out * nb * 64u + (uint64_t)row0 * nb * 2u, 8 * nb * 2, full);
                }
            } else if (lane == 0) {
                const uint8_t *mat = a.w0.data + (uint64_t)grp.expert * a.w0.expert_bytes;
                tbar_expect(full, 16 * row_bytes + (LUT ? 16 * nb * 2 : 0));
                tbulk(stage, mat + (uint64_t)row0 * row_bytes, 16 * row_bytes, full);
                if (LUT) tbulk(stage + 4096, mat + (uint64_t)n_out * nb * 64u + (uint64_t)row0 * nb * 2u, 16 * nb * 2, full);
            }
        };
        const uint32_t slices = mine * spu;
        tproxy_fence();
        if (alive) for (uint32_t n = 0; n < TNS && n < slices; n++) issue(n);     // weights do not wait for the digits
        // the tokens of the group as this lane sees them in the epilogue: pair and scale of token 4q + t
        uint32_t pair_t[TNT];
        float xs[TNT], f[TNT][2];
#pragma unroll
        for (int q = 0; q < TNT; q++) {
            pair_t[q] = __shfl_sync(0xffffffffu, my_pair, (4 * q + t) & 31u);
            const uint32_t row_t = __shfl_sync(0xffffffffu, my_row, (4 * q + t) & 31u);
            xs[q] = 4u * q + t < count ? __ldg(a.scale + row_t) : 0.0f;
        }
        if (alive) alive = tbar_wait(digitbar, turn & 1u, a.status);
#pragma unroll 1
        for (uint32_t n = 0; n < slices; n++) {
            const uint32_t s = n % spu, at = ring_base + n;
            if (s == 0) {
#pragma unroll
                for (int q = 0; q < TNT; q++) f[q][0] = f[q][1] = 0.0f;
            }
            if (alive) alive = tbar_wait(&bar[at % TNS], (at / TNS) & 1u, a.status);
            alive = __all_sync(0xffffffffu, alive);
            const uint8_t *stage = ring + (at % TNS) * STAGE;
            if (alive) {
                RowView v;
                v.swz = iq2_swizzle(g, nb);
                v.aux0 = v.aux1 = v.dd0 = v.dd1 = nullptr;
                if (TYPE == T_Q2_K) {
                    const uint32_t per_row = MODE == 0 ? SB : nb;              // blocks of a row inside the stage
                    v.r0 = stage + g * per_row * 64u; v.r1 = stage + (8 + g) * per_row * 64u;
                    v.aux0 = stage + 4096 + g * per_row * 16u; v.aux1 = stage + 4096 + (8 + g) * per_row * 16u;
                    v.dd0 = stage + 5120 + g * per_row * 4u; v.dd1 = stage + 5120 + (8 + g) * per_row * 4u;
                    TileHalves<TYPE>::run(v, per_row * 2, MODE == 0 ? s * SB * 2 : 0, lut, t, bl, 8 * kp, n_tiles, f);
                } else if (MODE == 0) {
                    constexpr uint32_t slice_bytes = SB * BB;
                    v.r0 = stage + g * slice_bytes; v.r1 = stage + (8 + g) * slice_bytes;
                    v.dd0 = stage + 16 * slice_bytes + (g * nb + s * SB) * 2u; v.dd1 = stage + 16 * slice_bytes + ((8 + g) * nb + s * SB) * 2u;
                    TileHalves<TYPE>::run(v, SB * 2, s * SB * 2, lut, t, bl, 8 * kp, n_tiles, f);
                } else {
                    v.r0 = stage + g * row_bytes; v.r1 = stage + (8 + g) * row_bytes;
                    v.dd0 = stage + 4096 + g * nb * 2u; v.dd1 = stage + 4096 + (8 + g) * nb * 2u;
                    TileHalves<TYPE>::run(v, nb * 2, 0, lut, t, bl, 8 * kp, n_tiles, f);
                }
            }
            __syncwarp();
            tproxy_fence();
            if (alive && n + TNS < slices) issue(n + TNS);
            if (s + 1 == spu && alive) {                                       // tile complete
                const uint32_t tile = tile0 + (n / spu) * tile_step;
#pragma unroll
                for (int q = 0; q < TNT; q++) {
                    if (4u * q + t < count) {
                        const float v0 = f[q][0] * xs[q], v1 = f[q][1] * xs[q];
                        if (MODE == 0) {
                            const float e = __expf(-fabsf(v0));
                            const float sig = v0 >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
                            const float val = v0 * sig * v1;
                            if ((__float_as_uint(val) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                            a.out[(uint64_t)pair_t[q] * n_out + tile * 8 + g] = val;
                        } else {
                            if ((__float_as_uint(v0) & 0x7f800000u) == 0x7f800000u || (__float_as_uint(v1) & 0x7f800000u) == 0x7f800000u)
                                atomicOr(a.status, QW4SH_ERR_NONFINITE);
                            a.out[(uint64_t)pair_t[q] * n_out + tile * 16 + g] = v0;
                            a.out[(uint64_t)pair_t[q] * n_out + tile * 16 + 8 + g] = v1;
                        }
                    }
                }
            }
        }
        if (alive) ring_base += slices;
    }
}

// Groups of at most TROWS rows out of the expert-sorted lists.  One CTA, thread i owns active expert i (then i + 1024,
// ...); a block-wide exclusive scan of the group counts gives every expert its place in the list: active experts in
// ascending order, each expert's groups by ascending row.
__global__ void __launch_bounds__(1024) build_tile_groups_kernel(const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ active,
                                                                 TGroup *groups, uint32_t *n_groups) {
    __shared__ uint32_t wsum[32];
    __shared__ uint32_t s_base;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, n_active = active[0];
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (uint32_t i0 = 0; i0 < n_active; i0 += 1024) {
        const uint32_t i = i0 + tid;
        uint32_t e = 0, first = 0, end = 0;
        if (i < n_active) { e = active[1 + i]; first = offsets[e]; end = offsets[e + 1]; }
        const uint32_t count = (end - first + TROWS - 1) / TROWS;
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
        for (uint32_t r = first; r < end; r += TROWS) groups[at++] = TGroup{e, r, min(TROWS, end - r), 0};
        __syncthreads();
        if (tid == 1023) s_base = at;                                // end of the last thread = end of this pass
        __syncthreads();
    }
    if (tid == 0) *n_groups = s_base;
}
__global__ void build_dense_tile_groups_kernel(uint32_t tokens, TGroup *groups, uint32_t *n_groups) {
    const uint32_t n = (tokens + TROWS - 1) / TROWS;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        groups[i] = TGroup{0, i * TROWS, min(TROWS, tokens - i * TROWS), 0};
    if (blockIdx.x == 0 && threadIdx.x == 0) *n_groups = n;
}

}  // namespace qw4

using namespace qw4;

extern "C" int qw4sh_note_launch(const char *name);
extern "C" const uint8_t *qw4sh_lut_image(void);

static DevTensor tdev(const QW4ShTensor &s) {
    DevTensor t;
    t.data = s.data; t.type = s.type; t.k_storage = s.k_storage; t.k_logical = s.k_logical;
    t.n_out = s.n_out; t.n_experts = s.n_experts; t.row_bytes = s.row_bytes; t.expert_bytes = s.expert_bytes;
    return t;
}

extern "C" int qw4sh_tile_supported(const QW4ShTensor *w, int mode) {
    if (w->type != T_Q4_K && w->type != T_IQ2_XXS && w->type != T_Q2_K) return 0;
    if (w->k_storage % 256 || w->k_logical != w->k_storage) return 0;
    if (mode == 0) {
        if (w->k_storage % 1024 || w->k_storage > 4096 || w->n_out % 8) return 0;       // whole slices; super-scales of a unit fit the stage
    } else {
        if (w->n_out % 16 || (w->type == T_Q4_K ? w->k_storage > 512 : w->k_storage > 1024)) return 0;   // a 16-row tile fits one stage
    }
    const uint32_t smem = w->type == T_Q4_K ? tile_smem_bytes<T_Q4_K>(w->k_storage)
                        : w->type == T_Q2_K ? tile_smem_bytes<T_Q2_K>(w->k_storage) : tile_smem_bytes<T_IQ2_XXS>(w->k_storage);
    return smem <= 227u * 1024u;
}

// Groups of <= 16 rows (16-byte records {expert, first row, rows, 0}) for qw4sh_expert_tiles: from the expert-sorted
// lists, or dense (the shared expert: rows in token order).
extern "C" int qw4sh_build_tile_groups(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream) {
    build_tile_groups_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(offsets, active, (TGroup *)groups, n_groups);
    return qw4sh_note_launch("build_tile_groups_kernel");
}
extern "C" int qw4sh_build_dense_tile_groups(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream) {
    build_dense_tile_groups_kernel<<<(tokens / TROWS + 256) / 256, 256, 0, (cudaStream_t)stream>>>(tokens, (TGroup *)groups, n_groups);
    return qw4sh_note_launch("build_dense_tile_groups_kernel");
}

template <uint32_t TYPE, int MODE>
static int launch_tile(const TileArgs &a, const TileMaps &maps, int ctas, cudaStream_t stream) {
    const size_t smem = tile_smem_bytes<TYPE>(a.w0.k_storage);
    cudaError_t e = cudaFuncSetAttribute(expert_tile_kernel<TYPE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    expert_tile_kernel<TYPE, MODE><<<ctas, TT, smem, stream>>>(a, maps);
    return qw4sh_note_launch("expert_tile_kernel");
}

// ---- section maps of the gate / up tensors -------------------------------------------------------------------------
typedef CUresult (*TileEncode)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int section_map(const QW4ShTensor *t, uint64_t offset, uint32_t row_stride, uint32_t piece, CUtensorMap *map) {
    static TileEncode encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess || !fn) return -1;
        encode = (TileEncode)fn;
    }
    if (row_stride % 16 || piece % 16 || t->expert_bytes % 16 || ((uintptr_t)(t->data + offset) & 15u)) return -2;
    const cuuint64_t dims[3] = {row_stride / 4, t->n_out, t->n_experts};
    const cuuint64_t strides[2] = {row_stride, t->expert_bytes};
    const cuuint32_t box[3] = {piece / 4, 8, 1}, elem[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (void *)(t->data + offset), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}
// Called once the images are resident: the gate / up tensors (routed and shared) that the tile kernels can take get
// their section maps; a tensor without them is copied row by row.  Never fails the create.
extern "C" int qw4sh_tile_prepare(QW4ShLayer *l) {
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    const int which[4] = {1, 2, 4, 5};
    for (int i = 0; i < 4; i++) {
        QW4ShTensor *t = &l->w[which[i]];
        t->tile_sections = 0;
        if (!qw4sh_tile_supported(t, 0)) continue;
        const uint32_t nb = t->k_storage >> 8;
        const uint64_t blocks = (uint64_t)t->n_out * nb;
        alignas(64) CUtensorMap maps[3];
        int rc = 0, sections = 1;
        if (t->type == T_Q4_K) rc = section_map(t, 0, nb * 144u, TGeo<T_Q4_K>::SLICE_BLOCKS * 144u, &maps[0]);
        else if (t->type == T_IQ2_XXS) rc = section_map(t, 0, nb * 64u, TGeo<T_IQ2_XXS>::SLICE_BLOCKS * 64u, &maps[0]);
        else {
            constexpr uint32_t SB = TGeo<T_Q2_K>::SLICE_BLOCKS;
            sections = 3;
            rc = section_map(t, 0, nb * 64u, SB * 64u, &maps[0]);
            if (!rc) rc = section_map(t, blocks * 64u, nb * 16u, SB * 16u, &maps[1]);
            if (!rc) rc = section_map(t, blocks * 80u, nb * 4u, SB * 4u, &maps[2]);
        }
        if (rc) continue;
        memcpy(t->tile_maps, maps, sizeof(CUtensorMap) * sections);
        t->tile_sections = sections;
    }
    return 0;
}

// mode 0: gate (w0) + up (w1) -> act [pairs][n_out]; mode 1: down (w0) -> out [pairs][n_out].  Input rows are
// the quantised rows of quantize_rows (row = pair / k_div); groups are those of qw4sh_build_tile_groups /
// qw4sh_build_dense_tile_groups.
extern "C" int qw4sh_expert_tiles(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                                  const uint32_t *row_to_pair, uint32_t k_div, const int8_t *digits, const int *sums, const float *scale,
                                  float *out, uint32_t *status, int ctas, void *stream) {
    TileArgs a;
    a.w0 = tdev(*w0); a.w1 = tdev(w1 ? *w1 : *w0);
    a.groups = (const TGroup *)groups; a.n_groups = n_groups; a.row_to_pair = row_to_pair; a.k_div = k_div;
    a.digits = digits; a.sums = sums; a.scale = scale; a.lut = nullptr; a.out = out; a.status = status;
    if (w0->type == T_IQ2_XXS && !(a.lut = qw4sh_lut_image())) return -3;
    alignas(64) TileMaps maps;
    memset(&maps, 0, sizeof maps);
    const int want = w0->type == T_Q2_K ? 3 : 1;
    a.use_maps = mode == 0 && w1 && w0->tile_sections == want && w1->tile_sections == want ? 1u : 0u;
    if (a.use_maps) { memcpy(maps.m[0], w0->tile_maps, sizeof(CUtensorMap) * want); memcpy(maps.m[1], w1->tile_maps, sizeof(CUtensorMap) * want); }
    cudaStream_t s = (cudaStream_t)stream;
    if (w0->type == T_Q4_K) return mode == 0 ? launch_tile<T_Q4_K, 0>(a, maps, ctas, s) : launch_tile<T_Q4_K, 1>(a, maps, ctas, s);
    if (w0->type == T_Q2_K) return mode == 0 ? launch_tile<T_Q2_K, 0>(a, maps, ctas, s) : launch_tile<T_Q2_K, 1>(a, maps, ctas, s);
    return mode == 0 ? launch_tile<T_IQ2_XXS, 0>(a, maps, ctas, s) : launch_tile<T_IQ2_XXS, 1>(a, maps, ctas, s);
}
