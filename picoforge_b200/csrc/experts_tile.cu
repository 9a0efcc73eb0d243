// Expert products for mid-sized groups (up to 32 token rows per group) on the int8 tensor-core
// path, with each weight fragment built ONCE and applied to all of the group's 4-token column tiles.
//
// Between the one-kernel decode path (<= 4 tokens) and the tcgen05 grouped GEMM (dense groups)
// lies the regime of batched decode and sparse prefill: an expert sees a handful to a few dozen
// rows.  A tcgen05.mma costs the same 144 cycles whatever its N, so few rows waste it; here the
// cost per weight is the fragment build plus about a dozen instructions per column tile.
//
// A work unit is (group of <= 32 rows of one expert, row tile): gate/up tiles are 8 gate rows + the
// same 8 up rows (MMA rows 0-7 and 8-15, so SwiGLU stays in the lane), down tiles 16 rows.  One
// warp owns a unit: it streams the tile's packed rows slice by slice with TMA bulk copies into its
// own two-stage ring and runs mma.sync.m16n8k32.s8 on the raw codes against the two-int8-digit
// images of the activations (quantize_rows), which it reads straight from global memory: a
// group's digits are shared by all of its tiles and stay in L1 / L2.  No cross-warp reduction, no
// CTA barrier after the prologue.
//
// Every mbarrier wait is bounded (about a second) and then records QW4SH_ERR_STATE.
#include <cuda_runtime.h>
#include <stdint.h>

#include "cuda_shim.h"
#include "formats.cuh"

namespace qw4 {

constexpr int TW = 12;                          // warps per CTA (168 registers each: room to run the digit loads ahead)
constexpr int TT = TW * 32;
constexpr int TNS = 2;                          // ring stages per warp
constexpr uint32_t TSTAGE = 5376;               // bytes per stage (Q2_K: 4096 codes + 1024 scale bytes + 256 super-scales)
constexpr int TNT = 8;                          // column tiles per group (32 rows)
constexpr uint32_t T_LUT_GRID = 256 * 128, T_LUT_SIGN = 128 * 128, T_LUT_BYTES = T_LUT_GRID + T_LUT_SIGN;

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
};

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
__device__ __forceinline__ void tproxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmma_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <uint32_t TYPE> struct TGeo;
template <> struct TGeo<T_Q4_K> { static constexpr uint32_t SLICE_BLOCKS = 2, BLOCK_BYTES = 144; };
template <> struct TGeo<T_IQ2_XXS> { static constexpr uint32_t SLICE_BLOCKS = 4, BLOCK_BYTES = 64; };
template <> struct TGeo<T_Q2_K> { static constexpr uint32_t SLICE_BLOCKS = 4, BLOCK_BYTES = 64; };       // codes; scale bytes and super-scales apart

// The lane's view of a group's activations: for column tile n, `bq[n]` is the byte offset of the
// digit row of MMA column g (token 4n + g / 2, digit g & 1) at this lane's 8-column phase, `xs[n]`
// the scale of token 4n + t.
struct LaneTokens {
    uint32_t bq[TNT];
    float xs[TNT];
};

// The two rows of a lane inside a ring stage: packed codes, and where the format keeps them apart its
// sub-block scale bytes (Q2_K) and super-scales (IQ2_XXS: fp16 d per block; Q2_K: {d, dmin} per block).
struct RowView {
    const uint8_t *r0, *r1, *aux0, *aux1, *dd0, *dd1;
    uint32_t swz;                                // IQ2_XXS: group swizzle of these rows
};

// The B operands (activation digits) come straight from global memory: lane (g, t) reads the eight bytes of MMA
// column g (token 4n + g / 2, digit g & 1) at its column phase, for every column tile n.  To keep those loads off
// the critical path each 128-byte line (one half block of one digit row) is brought into L1 one half block ahead
// with prefetch.global.L1, and the fragments of chunk j + 1 are loaded into registers before the MMAs of chunk j.
__device__ __forceinline__ void load_b(uint2 (&b)[TNT], const int8_t *digits, const LaneTokens &lt, uint32_t tiles, uint32_t col) {
#pragma unroll
    for (int n = 0; n < TNT; n++)
        b[n] = (uint32_t)n < tiles ? __ldg(reinterpret_cast<const uint2 *>(digits + lt.bq[n] + col)) : make_uint2(0u, 0u);
}
__device__ __forceinline__ void prefetch_b(const int8_t *digits, const LaneTokens &lt, uint32_t tiles, uint32_t col) {
#pragma unroll
    for (int n = 0; n < TNT; n++)
        if ((uint32_t)n < tiles) asm volatile("prefetch.global.L1 [%0];" ::"l"(digits + lt.bq[n] + col));
}

// One span of `halves` half blocks (128 columns each) of rows r0 / r1 against every column tile; the span starts at
// half block `first_half` of a row of `row_halves`.
// f[n][0] += row g . x[token 4n + t], f[n][1] += row g + 8 . x[token 4n + t] (in digit units).
template <uint32_t TYPE> struct TileHalves;

// Q4_K: the 4-bit codes are the A operand; the 6-bit sub-block minimum goes through a second MMA whose A operand
// is the minimum replicated over the lane's columns, so both sums come out of the tensor core.
template <> struct TileHalves<T_Q4_K> {
    static __device__ __forceinline__ void run(const RowView &v, uint32_t halves, uint32_t first_half, uint32_t row_halves, const uint8_t *,
                                               uint32_t t, const int8_t *digits, const LaneTokens &lt, uint32_t tiles, float (&f)[TNT][2]) {
        const uint8_t *r0 = v.r0, *r1 = v.r1;
        const float lo = 1.0f / 254.0f;
        uint2 bc[TNT], bn[TNT];
        load_b(bc, digits, lt, tiles, first_half * 128u);
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++) {
            const uint8_t *b0 = r0 + (h >> 1) * 144u, *b1 = r1 + (h >> 1) * 144u;
            const uint32_t hb = h & 1u, col0 = (first_half + h) * 128u;
            if (first_half + h + 1 < row_halves) prefetch_b(digits, lt, tiles, col0 + 128u);
            const uint4 h0 = *reinterpret_cast<const uint4 *>(b0), h1 = *reinterpret_cast<const uint4 *>(b1);
            uint32_t sc0, mn0, sc1, mn1;
            if (hb == 0) { sc0 = h0.y & 0x3f3f3f3fu; mn0 = h0.z & 0x3f3f3f3fu; sc1 = h1.y & 0x3f3f3f3fu; mn1 = h1.z & 0x3f3f3f3fu; }
            else {
                sc0 = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u); mn0 = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u);
                sc1 = (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u); mn1 = ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u);
            }
            const float d0 = __half2float(__ushort_as_half((uint16_t)(h0.x & 0xffffu))), n0 = __half2float(__ushort_as_half((uint16_t)(h0.x >> 16)));
            const float d1 = __half2float(__ushort_as_half((uint16_t)(h1.x & 0xffffu))), n1 = __half2float(__ushort_as_half((uint16_t)(h1.x >> 16)));
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const uint2 q0 = *reinterpret_cast<const uint2 *>(b0 + 16 + (hb * 2 + cc) * 32 + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(b1 + 16 + (hb * 2 + cc) * 32 + 8 * t);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int j = cc * 2 + nib;
                    if (j < 3) load_b(bn, digits, lt, tiles, col0 + (j + 1) * 32u);
                    else if (h + 1 < halves) load_b(bn, digits, lt, tiles, col0 + 128u);
                    const uint32_t a0 = (q0.x >> (4 * nib)) & 0x0f0f0f0fu, a1 = (q1.x >> (4 * nib)) & 0x0f0f0f0fu;
                    const uint32_t a2 = (q0.y >> (4 * nib)) & 0x0f0f0f0fu, a3 = (q1.y >> (4 * nib)) & 0x0f0f0f0fu;
                    const float ds0 = d0 * (float)((sc0 >> (8 * j)) & 0xffu), ds1 = d1 * (float)((sc1 >> (8 * j)) & 0xffu);
                    const uint32_t m0 = ((mn0 >> (8 * j)) & 0xffu) * 0x01010101u, m1 = ((mn1 >> (8 * j)) & 0xffu) * 0x01010101u;
#pragma unroll
                    for (int n = 0; n < TNT; n++) {
                        if ((uint32_t)n < tiles) {
                            int c[4], e[4];
                            tmma_zero(c, a0, a1, a2, a3, bc[n].x, bc[n].y);
                            tmma_zero(e, m0, m1, m0, m1, bc[n].x, bc[n].y);
                            f[n][0] += ds0 * fmaf((float)c[1], lo, (float)c[0]) - n0 * fmaf((float)e[1], lo, (float)e[0]);
                            f[n][1] += ds1 * fmaf((float)c[3], lo, (float)c[2]) - n1 * fmaf((float)e[3], lo, (float)e[2]);
                        }
                    }
#pragma unroll
                    for (int n = 0; n < TNT; n++) bc[n] = bn[n];
                }
            }
        }
    }
};

template <> struct TileHalves<T_IQ2_XXS> {
    static __device__ __forceinline__ void run(const RowView &v, uint32_t halves, uint32_t first_half, uint32_t row_halves, const uint8_t *lut,
                                               uint32_t t, const int8_t *digits, const LaneTokens &lt, uint32_t tiles, float (&f)[TNT][2]) {
        const uint8_t *r0 = v.r0, *r1 = v.r1;
        const uint16_t *d0p = reinterpret_cast<const uint16_t *>(v.dd0), *d1p = reinterpret_cast<const uint16_t *>(v.dd1);
        const uint32_t swz = v.swz;
        const uint8_t *grid = lut + (threadIdx.x & 15u) * 8u;
        const uint8_t *sign = lut + T_LUT_GRID + (threadIdx.x & 7u) * 16u;
        const uint32_t pick = 0x4440u + t, shift_s = 7 * t;
        const float lo = 1.0f / 254.0f;
        uint2 bc[TNT], bn[TNT];
        load_b(bc, digits, lt, tiles, first_half * 128u);
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++) {
            const uint32_t at = ((h * 4u) ^ swz) * 8u, col0 = (first_half + h) * 128u;
            if (first_half + h + 1 < row_halves) prefetch_b(digits, lt, tiles, col0 + 128u);
            const float d0 = __half2float(__ushort_as_half(d0p[h >> 1])) * 0.125f, d1 = __half2float(__ushort_as_half(d1p[h >> 1])) * 0.125f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (j < 3) load_b(bn, digits, lt, tiles, col0 + (j + 1) * 32u);
                else if (h + 1 < halves) load_b(bn, digits, lt, tiles, col0 + 128u);
                const uint2 g0 = *reinterpret_cast<const uint2 *>(r0 + at + 8 * j), g1 = *reinterpret_cast<const uint2 *>(r1 + at + 8 * j);
                const uint32_t i0 = __byte_perm(g0.x, 0u, pick), i1 = __byte_perm(g1.x, 0u, pick);
                const uint32_t s0 = (g0.y >> shift_s) & 127u, s1 = (g1.y >> shift_s) & 127u;
                const uint2 v0 = *reinterpret_cast<const uint2 *>(grid + i0 * 128u), v1 = *reinterpret_cast<const uint2 *>(grid + i1 * 128u);
                const uint4 m0 = *reinterpret_cast<const uint4 *>(sign + s0 * 128u), m1 = *reinterpret_cast<const uint4 *>(sign + s1 * 128u);
                const uint32_t a0 = (v0.x ^ m0.x) + m0.z, a1 = (v1.x ^ m1.x) + m1.z, a2 = (v0.y ^ m0.y) + m0.w, a3 = (v1.y ^ m1.y) + m1.w;
                const float ds0 = d0 * (float)((g0.y >> 27) | 1u), ds1 = d1 * (float)((g1.y >> 27) | 1u);
#pragma unroll
                for (int n = 0; n < TNT; n++) {
                    if ((uint32_t)n < tiles) {
                        int c[4];
                        tmma_zero(c, a0, a1, a2, a3, bc[n].x, bc[n].y);
                        f[n][0] += ds0 * fmaf((float)c[1], lo, (float)c[0]);
                        f[n][1] += ds1 * fmaf((float)c[3], lo, (float)c[2]);
                    }
                }
#pragma unroll
                for (int n = 0; n < TNT; n++) bc[n] = bn[n];
            }
        }
    }
};

// Q2_K in the resident image: 64 code bytes per block, 16 scale/min bytes per block, one word {d, dmin} per
// block, each in its own section.  A 32-column chunk
// spans two 16-column sub-blocks; lane (g, t) holds eight columns of ONE sub-block, so the 4-bit sub-block scale is
// multiplied into the 2-bit codes (<= 45, still int8) and the minimum goes through a second MMA whose A operand is
// the minimum replicated over the lane's columns: both sums come out of the tensor core, no per-16-column digit
// sums needed.
template <> struct TileHalves<T_Q2_K> {
    static __device__ __forceinline__ void run(const RowView &v, uint32_t halves, uint32_t first_half, uint32_t row_halves, const uint8_t *,
                                               uint32_t t, const int8_t *digits, const LaneTokens &lt, uint32_t tiles, float (&f)[TNT][2]) {
        const float lo = 1.0f / 254.0f;
        const uint8_t *r0 = v.r0, *r1 = v.r1, *s0 = v.aux0, *s1 = v.aux1;
        uint2 bc[TNT], bn[TNT];
        load_b(bc, digits, lt, tiles, first_half * 128u);
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++) {
            const uint32_t blk = h >> 1, hb = h & 1u, col0 = (first_half + h) * 128u;
            if (first_half + h + 1 < row_halves) prefetch_b(digits, lt, tiles, col0 + 128u);
            const uint2 q0 = *reinterpret_cast<const uint2 *>(r0 + blk * 64u + hb * 32u + 8u * t);
            const uint2 q1 = *reinterpret_cast<const uint2 *>(r1 + blk * 64u + hb * 32u + 8u * t);
            const uint2 w0 = *reinterpret_cast<const uint2 *>(s0 + blk * 16u + hb * 8u), w1 = *reinterpret_cast<const uint2 *>(s1 + blk * 16u + hb * 8u);
            const uint32_t dd0 = *reinterpret_cast<const uint32_t *>(v.dd0 + blk * 4u), dd1 = *reinterpret_cast<const uint32_t *>(v.dd1 + blk * 4u);
            const float d0 = __half2float(__ushort_as_half((uint16_t)(dd0 & 0xffffu))), n0 = __half2float(__ushort_as_half((uint16_t)(dd0 >> 16)));
            const float d1 = __half2float(__ushort_as_half((uint16_t)(dd1 & 0xffffu))), n1 = __half2float(__ushort_as_half((uint16_t)(dd1 >> 16)));
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (j < 3) load_b(bn, digits, lt, tiles, col0 + (j + 1) * 32u);
                else if (h + 1 < halves) load_b(bn, digits, lt, tiles, col0 + 128u);
                const uint32_t sh = 8u * ((j & 1) * 2 + (t >> 1));
                const uint32_t b0 = ((j < 2 ? w0.x : w0.y) >> sh) & 0xffu, b1 = ((j < 2 ? w1.x : w1.y) >> sh) & 0xffu;
                const uint32_t sc0 = b0 & 15u, sc1 = b1 & 15u, m0 = (b0 >> 4) * 0x01010101u, m1 = (b1 >> 4) * 0x01010101u;
                const uint32_t a0 = ((q0.x >> (2 * j)) & 0x03030303u) * sc0, a1 = ((q1.x >> (2 * j)) & 0x03030303u) * sc1;
                const uint32_t a2 = ((q0.y >> (2 * j)) & 0x03030303u) * sc0, a3 = ((q1.y >> (2 * j)) & 0x03030303u) * sc1;
#pragma unroll
                for (int n = 0; n < TNT; n++) {
                    if ((uint32_t)n < tiles) {
                        int c[4], e[4];
                        tmma_zero(c, a0, a1, a2, a3, bc[n].x, bc[n].y);
                        tmma_zero(e, m0, m1, m0, m1, bc[n].x, bc[n].y);
                        f[n][0] += d0 * fmaf((float)c[1], lo, (float)c[0]) - n0 * fmaf((float)e[1], lo, (float)e[0]);
                        f[n][1] += d1 * fmaf((float)c[3], lo, (float)c[2]) - n1 * fmaf((float)e[3], lo, (float)e[2]);
                    }
                }
#pragma unroll
                for (int n = 0; n < TNT; n++) bc[n] = bn[n];
            }
        }
    }
};

// MODE 0: gate + up + SwiGLU -> act; MODE 1: down -> out.
template <uint32_t TYPE, int MODE>
__global__ void __launch_bounds__(TT, 1) expert_tile_kernel(const TileArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool LUT = TYPE == T_IQ2_XXS;
    constexpr uint32_t SB = TGeo<TYPE>::SLICE_BLOCKS, BB = TGeo<TYPE>::BLOCK_BYTES;
    uint64_t *ringbar = reinterpret_cast<uint64_t *>(smem);                    // [TW][TNS], then the table barrier
    uint64_t *lutbar = ringbar + TW * TNS;
    const uint8_t *lut = smem + 512;
    uint8_t *rings = smem + 512 + (LUT ? T_LUT_BYTES : 0);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t K = a.w0.k_storage, nb = K >> 8, n_out = a.w0.n_out;
    const uint32_t tile_rows = MODE == 0 ? 8u : 16u, tiles = n_out / tile_rows;
    const uint32_t row_bytes = nb * BB;                                        // Q4_K, IQ2_XXS payload (Q2_K: code bytes)
    // MODE 0 streams K in slices; MODE 1 fetches a whole 16-row tile (K <= 512 for Q4_K, <= 1024 for IQ2_XXS)
    const uint32_t spu = MODE == 0 ? nb / SB : 1u;
    if (tid == 0) {
        for (uint32_t i = 0; i < TW * TNS; i++) tbar_init(&ringbar[i], 1);
        tbar_init(lutbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (LUT && tid == 0) {
        tbar_expect(lutbar, T_LUT_BYTES);
        tbulk(smem + 512, a.lut, T_LUT_BYTES, lutbar);
    }
    const uint32_t n_groups = *a.n_groups;
    const uint32_t total = n_groups * tiles;
    // a CTA takes runs of consecutive units (mostly one group: its digits stay in this SM's L1); with few units
    // the runs shrink so that every SM gets some
    const uint32_t run = min((uint32_t)TW, (total + gridDim.x - 1) / gridDim.x);
    if (warp >= run) return;
    const uint32_t blocks = (total + run - 1) / run;
    uint32_t mine = 0;
    for (uint32_t b = blockIdx.x; b < blocks; b += gridDim.x) mine += b * run + warp < total ? 1u : 0u;
    if (!mine) return;
    uint8_t *ring = rings + warp * TNS * TSTAGE;
    uint64_t *bar = ringbar + warp * TNS;
    bool alive = true;
    if (LUT) alive = tbar_wait(lutbar, 0, a.status);
    const uint32_t slices = mine * spu;
    auto unit_of = [&](uint32_t i) { return (blockIdx.x + i * gridDim.x) * run + warp; };
    auto issue = [&](uint32_t n) {
        const uint32_t u = unit_of(n / spu), s = n % spu;
        const TGroup grp = a.groups[u / tiles];
        const uint32_t row0 = (u % tiles) * tile_rows;
        uint8_t *stage = ring + (n % TNS) * TSTAGE;
        uint64_t *full = &bar[n % TNS];
        if (TYPE == T_Q2_K) {
            // three sections per matrix: codes, scale bytes, {d, dmin}; in the stage at 0, 4096 and 5120
            const uint64_t blocks = (uint64_t)n_out * nb;
            if (MODE == 0) {
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
    if (alive) for (uint32_t n = 0; n < TNS && n < slices; n++) issue(n);
    LaneTokens lt;
    uint32_t pair_t[TNT];                                                      // pair of token 4n + t
    float f[TNT][2];
    uint32_t n_tiles = 0, count = 0;
#pragma unroll 1
    for (uint32_t n = 0; n < slices; n++) {
        const uint32_t u = unit_of(n / spu), s = n % spu;
        if (s == 0) {                                                          // new unit: the group's tokens as this lane sees them
            const TGroup grp = a.groups[u / tiles];
            count = grp.count; n_tiles = (count + 3) >> 2;
            uint32_t my_pair = 0;
            if (lane < count) my_pair = a.row_to_pair ? a.row_to_pair[grp.first + lane] : grp.first + lane;
            const uint32_t my_row = my_pair / a.k_div;
#pragma unroll
            for (int q = 0; q < TNT; q++) {
                const uint32_t row_g = __shfl_sync(0xffffffffu, my_row, (4 * q + (g >> 1)) & 31u);     // rows beyond the group read row 0's digits
                const uint32_t row_t = __shfl_sync(0xffffffffu, my_row, (4 * q + t) & 31u);
                pair_t[q] = __shfl_sync(0xffffffffu, my_pair, (4 * q + t) & 31u);
                lt.bq[q] = (row_g * 2 + (g & 1u)) * K + 8 * t;
                lt.xs[q] = (uint32_t)q < n_tiles ? __ldg(a.scale + row_t) : 0.0f;
                f[q][0] = f[q][1] = 0.0f;
            }
        }
        if (alive) alive = tbar_wait(&bar[n % TNS], (n / TNS) & 1u, a.status);
        alive = __all_sync(0xffffffffu, alive);
        const uint8_t *stage = ring + (n % TNS) * TSTAGE;
        if (alive) {
            RowView v;
            v.swz = iq2_swizzle(g, nb);
            v.aux0 = v.aux1 = v.dd0 = v.dd1 = nullptr;
            if (TYPE == T_Q2_K) {
                const uint32_t per_row = MODE == 0 ? SB : nb;                  // blocks of a row inside the stage
                v.r0 = stage + g * per_row * 64u; v.r1 = stage + (8 + g) * per_row * 64u;
                v.aux0 = stage + 4096 + g * per_row * 16u; v.aux1 = stage + 4096 + (8 + g) * per_row * 16u;
                v.dd0 = stage + 5120 + g * per_row * 4u; v.dd1 = stage + 5120 + (8 + g) * per_row * 4u;
                TileHalves<TYPE>::run(v, per_row * 2, MODE == 0 ? s * SB * 2 : 0, nb * 2, lut, t, a.digits, lt, n_tiles, f);
            } else if (MODE == 0) {
                constexpr uint32_t slice_bytes = SB * BB;
                v.r0 = stage + g * slice_bytes; v.r1 = stage + (8 + g) * slice_bytes;
                v.dd0 = stage + 16 * slice_bytes + (g * nb + s * SB) * 2u; v.dd1 = stage + 16 * slice_bytes + ((8 + g) * nb + s * SB) * 2u;
                TileHalves<TYPE>::run(v, SB * 2, s * SB * 2, nb * 2, lut, t, a.digits, lt, n_tiles, f);
            } else {
                v.r0 = stage + g * row_bytes; v.r1 = stage + (8 + g) * row_bytes;
                v.dd0 = stage + 4096 + g * nb * 2u; v.dd1 = stage + 4096 + (8 + g) * nb * 2u;
                TileHalves<TYPE>::run(v, nb * 2, 0, nb * 2, lut, t, a.digits, lt, n_tiles, f);
            }
        }
        __syncwarp();
        tproxy_fence();
        if (alive && n + TNS < slices) issue(n + TNS);
        if (s + 1 == spu && alive) {                                           // unit complete
            const uint32_t tile = u % tiles;
#pragma unroll
            for (int q = 0; q < TNT; q++) {
                if (4u * q + t < count) {
                    const float v0 = f[q][0] * lt.xs[q], v1 = f[q][1] * lt.xs[q];
                    if (MODE == 0) {
                        const float e = __expf(-fabsf(v0));
                        const float sig = v0 >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
                        const float v = v0 * sig * v1;
                        if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                        a.out[(uint64_t)pair_t[q] * n_out + tile * 8 + g] = v;
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
    return 1;
}

template <uint32_t TYPE, int MODE>
static int launch_tile(const TileArgs &a, int ctas, cudaStream_t stream) {
    const size_t smem = 512 + (TYPE == T_IQ2_XXS ? T_LUT_BYTES : 0) + (size_t)TW * TNS * TSTAGE;
    cudaError_t e = cudaFuncSetAttribute(expert_tile_kernel<TYPE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    expert_tile_kernel<TYPE, MODE><<<ctas, TT, smem, stream>>>(a);
    return qw4sh_note_launch("expert_tile_kernel");
}

// mode 0: gate (w0) + up (w1) -> act [pairs][n_out]; mode 1: down (w0) -> out [pairs][n_out].  Input rows are
// the quantised rows of quantize_rows (row = pair / k_div); groups are the 16-byte records of qw4sh_build_groups32 /
// qw4sh_build_dense_groups32 (<= 32 rows each).
extern "C" int qw4sh_expert_tiles(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                                  const uint32_t *row_to_pair, uint32_t k_div, const int8_t *digits, const int *sums, const float *scale,
                                  float *out, uint32_t *status, int ctas, void *stream) {
    TileArgs a;
    a.w0 = tdev(*w0); a.w1 = tdev(w1 ? *w1 : *w0);
    a.groups = (const TGroup *)groups; a.n_groups = n_groups; a.row_to_pair = row_to_pair; a.k_div = k_div;
    a.digits = digits; a.sums = sums; a.scale = scale; a.lut = nullptr; a.out = out; a.status = status;
    if (w0->type == T_IQ2_XXS && !(a.lut = qw4sh_lut_image())) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (w0->type == T_Q4_K) return mode == 0 ? launch_tile<T_Q4_K, 0>(a, ctas, s) : launch_tile<T_Q4_K, 1>(a, ctas, s);
    if (w0->type == T_Q2_K) return mode == 0 ? launch_tile<T_Q2_K, 0>(a, ctas, s) : launch_tile<T_Q2_K, 1>(a, ctas, s);
    return mode == 0 ? launch_tile<T_IQ2_XXS, 0>(a, ctas, s) : launch_tile<T_IQ2_XXS, 1>(a, ctas, s);
}
