// The whole MoE layer for a decode step of up to four tokens as ONE persistent kernel (sm_100a).
//
// One CTA per SM, launched cooperatively so that all CTAs are resident; two grid-wide barriers
// separate three phases (picoforge src/qwen4_moe.c:334-382 is the CPU statement of the sequence):
//
//   A  every CTA stages x, turns it into int8 digit pairs, and computes its 3-4 rows of the
//      router projection (plus the shared expert's gate row): exact mode walks k = 0..K-1 with
//      separately rounded products and sums (the reference's bits, src/qwen4_packed.c:164-173),
//      fast mode uses warp-tree sums.  The shared expert's tensors are prefetched into L2.
//   B  every CTA routes all tokens itself from the logits (softmax, top-k, renormalise; the same
//      arithmetic in every CTA, so no second exchange is needed), builds the list of distinct
//      experts, prefetches its down-projection tiles into L2, and streams its share of the
//      gate/up rows.  A work unit is 8 gate rows + the same 8 up rows of one expert (gate rows in
//      MMA rows 0-7, up rows in 8-15, so the lane that holds gate.x also holds up.x); a unit is cut
//      into K slices, and the CTA's slices are dealt to its warps round robin.  A warp fetches a
//      slice with TMA bulk copies into its own two-stage ring (no producer warp, no CTA-wide
//      barrier inside the stream), feeds int8 tensor-core MMAs with the raw codes and leaves its
//      partial sums in shared memory; after one CTA barrier the units are summed in slice order,
//      SwiGLU is applied and the result stored, with the row maxima kept for phase C.
//   C  CTA c owns 16 columns of y: its warps split the sources (shared expert + distinct routed
//      experts), each runs the 16 x K down tile on the tensor cores against the digit image of the
//      pair's activation, scales by the route weight (or the sigmoid gate) and the partial sums
//      are added in warp order: y is deterministic.
//
// The four tokens' digit pairs fill the eight MMA columns, so every expert sees the same B
// operand in phase B; results of tokens not routed to an expert are simply not stored.
//
// Code that runs once per launch is kept compact on purpose (loops instead of unrolled
// sequences, no per-thread arrays in local memory): a kernel of this kind executes most of its
// instructions a handful of times.
//
// Every wait (mbarrier or grid barrier) is bounded: after about a second the kernel records
// QW4SH_ERR_STATE and leaves.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "cuda_shim.h"
#include "formats.cuh"
#include "route.cuh"

namespace qw4 {

constexpr int FW = 12;                          // warps per CTA
constexpr int FT = FW * 32;
constexpr int FTOK = 4;                         // tokens per launch
constexpr int FMAXK = 16;                       // top-k limit
constexpr int FMAXE = 512;                      // experts limit
constexpr int FMAXSRC = FTOK * FMAXK + 1;       // shared expert + distinct routed experts
constexpr int FRMAX = 4;                        // router rows per CTA
constexpr int FRCH = 4;                         // router row chunks (one mbarrier each)
constexpr int FNS = 2;                          // ring stages per warp
constexpr uint32_t FSTAGE = 4608;               // bytes per ring stage (IQ2_XXS: 4096 payload + 512 super-scales)
constexpr uint32_t F_LUT_GRID = 256 * 128, F_LUT_SIGN = 128 * 128, F_LUT_BYTES = F_LUT_GRID + F_LUT_SIGN;
constexpr uint32_t F_SYNC_CLOCKS = 8, F_SYNC_AMAX = 64;   // word offsets inside the sync array

struct FusedArgs {
    DevTensor w[8];                             // router, gate, up, down, sgate, sup, sdown, srouter
    const float *x;
    float *y;
    uint32_t tokens, hidden, experts, top_k, inter, shared_inter;
    int norm, router_mode;
    float *logits, *shared_logit;               // [T, E], [T]
    uint32_t *ids;                              // [T, k]
    float *weights;                             // [T, k]
    float *act, *shared_act;                    // [T*k, I], [T, Is]
    uint32_t *ids_out;
    float *weights_out;
    const uint8_t *lut;                         // IQ2_XXS tables image (F_LUT_BYTES) or nullptr
    uint32_t *sync;                             // [0] barrier 1, [1] barrier 2, [2] exits, [8..39] clocks of CTA 0, [64..] row maxima
    uint32_t *status;
    uint32_t partial_slices;                    // capacity of the partial-sum buffer (slices per CTA)
};

// One distinct source of phase C / one expert of phase B.
struct Src {
    uint16_t expert; uint8_t mask, shared;
    uint32_t slots;                             // slot of token t in byte t
    __device__ __forceinline__ uint32_t slot(uint32_t t) const { return (slots >> (8 * t)) & 0xffu; }
};

// Shared-memory plan (byte offsets), the same on host and device.  `region` is reused by the
// three phases; the digit image of x lives at its start through phases A and B.
struct FPlan {
    uint32_t bars, ids, wts, misc, tokmask, slotmap, src, lut, region, total;
    uint32_t kp;                                // pitch of one digit row of x
    uint32_t xq, xsum;                          // phases A and B (inside region)
    uint32_t xf, xf_pitch, rows, row_pitch, prod;   // phase A
    uint32_t zs, ring, partial;                 // phase B
    uint32_t aq, ap, asum, ascale, aconst, tiles, cpartial;   // phase C
};
__host__ __device__ inline FPlan make_fplan(uint32_t hidden, uint32_t inter_max, uint32_t rows_c, uint32_t partial_slices, bool lut) {
    FPlan p;
    uint32_t at = 0;
    p.bars = at; at += 512;
    p.ids = at; at += FTOK * FMAXK * 4;
    p.wts = at; at += FTOK * FMAXK * 4;
    p.misc = at; at += 1024;                    // floats [0..3] x scales, [4..7] shared logits, [8..15] route scratch; words from +64;
                                                // +256: expf table (32 x 8 bytes); +512: digitiser constants of x (4 x float4)
    p.tokmask = at; at += FMAXE;
    p.slotmap = at; at += FMAXE * 4;
    p.src = at; at += ((FMAXSRC * 8 + 127) & ~127u);
    p.lut = at; if (lut) at += F_LUT_BYTES;
    p.region = at;
    p.kp = hidden + 32;
    uint32_t head = 0;
    p.xq = head; head += 8 * p.kp;
    p.xsum = head; head += FTOK * (hidden / 32) * 8;
    head = (head + 127) & ~127u;
    // phase A
    uint32_t a = head;
    p.xf_pitch = hidden * 4 + 16;
    p.xf = a; a += FTOK * p.xf_pitch;
    p.row_pitch = hidden * 4 + 16;
    p.rows = a; a += FRMAX * p.row_pitch;
    p.prod = a; a += 2 * 16 * (hidden / FRCH + 4) * 4;
    // phase B: the logits / probabilities are dead before the first copy lands in the ring
    uint32_t b = head;
    p.zs = b;
    p.ring = b; b += FW * FNS * FSTAGE;
    if (b < head + FTOK * FMAXE * 4) b = head + FTOK * FMAXE * 4;
    p.partial = b; b += partial_slices * 256;
    // phase C
    uint32_t c = 0;
    p.ap = inter_max + 32;
    p.aq = c; c += rows_c * 2 * p.ap;
    p.asum = c; c += rows_c * (inter_max / 32) * 8;
    p.ascale = c; c += ((rows_c * 4 + 127) & ~127u);
    p.aconst = c; c += ((rows_c * 16 + 127) & ~127u);
    c = (c + 127) & ~127u;
    p.tiles = c; c += FW * FNS * FSTAGE;
    p.cpartial = c; c += FW * 32 * 8;
    uint32_t m = a > b ? a : b;
    m = m > c ? m : c;
    p.total = p.region + m;
    return p;
}

// ---- small PTX helpers --------------------------------------------------------------------
__device__ __forceinline__ uint32_t fs_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fs_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fbar_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fs_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool fbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(fs_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait (about a second); false with the error bit set when it runs out.
__device__ __forceinline__ bool fbar_wait(uint64_t *bar, uint32_t parity, uint32_t *status) {
    if (fbar_try(bar, parity)) return true;
    const long long start = clock64();
    while (!fbar_try(bar, parity)) {
        if (clock64() - start > (1ll << 31)) { atomicOr(status, QW4SH_ERR_STATE); return false; }
    }
    return true;
}
__device__ __forceinline__ void fbulk(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(fs_u32(dst_smem)), "l"(src), "r"(bytes), "r"(fs_u32(bar)) : "memory");
}
__device__ __forceinline__ void fprefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fproxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t fld_acquire(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fmma_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// All CTAs arrive, then wait until `expected` have.  False (CTA-uniform) when the wait ran out.
__device__ __forceinline__ bool grid_barrier(uint32_t *counter, uint32_t expected, uint32_t *status, uint32_t *flag_smem) {
    __syncthreads();
    if (threadIdx.x == 0) {
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        uint32_t ok = 1;
        const long long start = clock64();
        while (fld_acquire(counter) < expected) {
            if (clock64() - start > (1ll << 31)) { atomicOr(status, QW4SH_ERR_STATE); ok = 0; break; }
        }
        *flag_smem = ok;
    }
    __syncthreads();
    return *flag_smem != 0;
}

// ---- half blocks (128 columns) on the tensor cores ----------------------------------------------
// MMA k-slots are permuted so that lane (g, t) owns the eight consecutive columns 8t..8t+7 of
// every 32-column chunk, for MMA rows g and g + 8 and for activation column g (token g >> 1,
// digit g & 1).  f0 += row g . x[token t], f1 += row g+8 . x[token t], both in units of the
// token's digit scale.  xq is the lane's digit pointer at the first chunk, xsum the token's digit
// sums (Q4_K's min term).
template <uint32_t TYPE> struct Halves;

// Q4_K: r0 / r1 point at the first 144-byte block of the two rows; `halves` half blocks follow.
template <> struct Halves<T_Q4_K> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, uint32_t halves, uint32_t, const uint16_t *,
                                            const uint16_t *, const uint8_t *, uint32_t t, const uint8_t *xq, const int2 *xsum,
                                            float &f0, float &f1) {
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++, xq += 128, xsum += 4) {
            const uint8_t *b0 = r0 + (h >> 1) * 144u, *b1 = r1 + (h >> 1) * 144u;
            const uint32_t hb = h & 1u;
            const uint4 h0 = *reinterpret_cast<const uint4 *>(b0), h1 = *reinterpret_cast<const uint4 *>(b1);
            uint32_t sc0, mn0, sc1, mn1;
            if (hb == 0) { sc0 = h0.y & 0x3f3f3f3fu; mn0 = h0.z & 0x3f3f3f3fu; sc1 = h1.y & 0x3f3f3f3fu; mn1 = h1.z & 0x3f3f3f3fu; }
            else {
                sc0 = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u); mn0 = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u);
                sc1 = (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u); mn1 = ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u);
            }
            int qacc[4] = {0, 0, 0, 0}, macc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {                             // 64 columns: low and high nibbles of 32 bytes
                const uint2 q0 = *reinterpret_cast<const uint2 *>(b0 + 16 + (hb * 2 + cc) * 32 + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(b1 + 16 + (hb * 2 + cc) * 32 + 8 * t);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int j = cc * 2 + nib;
                    const uint2 bq = *reinterpret_cast<const uint2 *>(xq + j * 32);
                    int c[4];
                    fmma_zero(c, (q0.x >> (4 * nib)) & 0x0f0f0f0fu, (q1.x >> (4 * nib)) & 0x0f0f0f0fu,
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
            f0 += d0 * fmaf((float)qacc[1], lo, (float)qacc[0]) - n0 * fmaf((float)macc[1], lo, (float)macc[0]);
            f1 += d1 * fmaf((float)qacc[3], lo, (float)qacc[2]) - n1 * fmaf((float)macc[3], lo, (float)macc[2]);
        }
    }
};

// IQ2_XXS: r0 / r1 point at the two rows' first 8-byte group of the span (a multiple of 16
// groups from the row start, so the in-row swizzle `swz` applies to the local index); d0p / d1p
// at the fp16 super-scales of the span's first block.
template <> struct Halves<T_IQ2_XXS> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, uint32_t halves, uint32_t swz, const uint16_t *d0p,
                                            const uint16_t *d1p, const uint8_t *lut, uint32_t t, const uint8_t *xq, const int2 *,
                                            float &f0, float &f1) {
        const uint8_t *grid = lut + (threadIdx.x & 15u) * 8u;            // 64-bit reads: 16 copies
        const uint8_t *sign = lut + F_LUT_GRID + (threadIdx.x & 7u) * 16u;   // 128-bit reads: 8 copies
        const uint32_t pick = 0x4440u + t, shift_s = 7 * t;
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++, xq += 128) {
            const uint32_t at = ((h * 4u) ^ swz) * 8u;
            int iacc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 g0 = *reinterpret_cast<const uint2 *>(r0 + at + 8 * j), g1 = *reinterpret_cast<const uint2 *>(r1 + at + 8 * j);
                const uint32_t i0 = __byte_perm(g0.x, 0u, pick), i1 = __byte_perm(g1.x, 0u, pick);
                const uint32_t s0 = (g0.y >> shift_s) & 127u, s1 = (g1.y >> shift_s) & 127u;
                const uint2 v0 = *reinterpret_cast<const uint2 *>(grid + i0 * 128u), v1 = *reinterpret_cast<const uint2 *>(grid + i1 * 128u);
                const uint4 m0 = *reinterpret_cast<const uint4 *>(sign + s0 * 128u), m1 = *reinterpret_cast<const uint4 *>(sign + s1 * 128u);
                const uint2 bq = *reinterpret_cast<const uint2 *>(xq + j * 32);
                int c[4];
                // m.x/m.y: 0xff where the weight is negative; m.z/m.w: 0x01 there.  Magnitudes are
                // never zero, so (v ^ 0xff) + 1 = -v stays inside its byte.
                fmma_zero(c, (v0.x ^ m0.x) + m0.z, (v1.x ^ m1.x) + m1.z, (v0.y ^ m0.y) + m0.w, (v1.y ^ m1.y) + m1.w, bq.x, bq.y);
                const int w0 = (int)((g0.y >> 27) | 1u), w1 = (int)((g1.y >> 27) | 1u);         // 2 * scale + 1
                iacc[0] += c[0] * w0; iacc[1] += c[1] * w0; iacc[2] += c[2] * w1; iacc[3] += c[3] * w1;
            }
            const float lo = 1.0f / 254.0f;
            const float d0 = __half2float(__ushort_as_half(d0p[h >> 1])) * 0.125f, d1 = __half2float(__ushort_as_half(d1p[h >> 1])) * 0.125f;
            f0 += d0 * fmaf((float)iacc[1], lo, (float)iacc[0]);
            f1 += d1 * fmaf((float)iacc[3], lo, (float)iacc[2]);
        }
    }
};

// Geometry of one format inside the rings.
template <uint32_t TYPE> struct FGeo;
template <> struct FGeo<T_Q4_K> { static constexpr uint32_t SLICE_BLOCKS = 2, BLOCK_BYTES = 144; };      // 512 columns, 288 B per row
template <> struct FGeo<T_IQ2_XXS> { static constexpr uint32_t SLICE_BLOCKS = 4, BLOCK_BYTES = 64; };    // 1024 columns, 256 B per row

// Copies of slice `s` of a gate/up unit (8 gate rows + 8 up rows from row `row0`) into `stage`:
// row r at r * slice bytes; IQ2_XXS also gets the unit's super-scales behind the rows.
template <uint32_t TYPE>
__device__ __forceinline__ void issue_unit_slice(const uint8_t *gate_mat, const uint8_t *up_mat, uint32_t n_out, uint32_t nb, uint32_t row0,
                                              uint32_t s, uint8_t *stage, uint64_t *bar, uint32_t lane) {
    const uint32_t row_bytes = nb * FGeo<TYPE>::BLOCK_BYTES;
    constexpr uint32_t slice_bytes = FGeo<TYPE>::SLICE_BLOCKS * FGeo<TYPE>::BLOCK_BYTES;
    if (lane == 0) fbar_expect(bar, 16 * slice_bytes + (TYPE == T_IQ2_XXS ? 2 * 8 * nb * 2 : 0));
    __syncwarp();
    if (lane < 16) {
        const uint8_t *mat = lane < 8 ? gate_mat : up_mat;
        fbulk(stage + lane * slice_bytes, mat + (row0 + (lane & 7u)) * row_bytes + s * slice_bytes, slice_bytes, bar);
    } else if (TYPE == T_IQ2_XXS && lane < 18) {
        const uint8_t *mat = lane == 16 ? gate_mat : up_mat;
        fbulk(stage + 16 * slice_bytes + (lane - 16) * 8 * nb * 2, mat + n_out * nb * 64u + row0 * nb * 2u, 8 * nb * 2, bar);
    }
}
template <uint32_t TYPE>
__device__ __forceinline__ void consume_unit_slice(const uint8_t *stage, uint32_t nb, uint32_t s, const uint8_t *lut, const uint8_t *xq_lane,
                                                   const int2 *xsum_tok, uint32_t g, uint32_t t, float &f0, float &f1) {
    constexpr uint32_t SB = FGeo<TYPE>::SLICE_BLOCKS, slice_bytes = SB * FGeo<TYPE>::BLOCK_BYTES;
    const uint16_t *d = reinterpret_cast<const uint16_t *>(stage + 16 * slice_bytes);
    Halves<TYPE>::run(stage + g * slice_bytes, stage + (8 + g) * slice_bytes, SB * 2, iq2_swizzle(g, nb), d + g * nb + s * SB,
                      d + (8 + g) * nb + s * SB, lut, t, xq_lane + s * SB * 256u, xsum_tok + s * SB * 8u, f0, f1);
}

// Down tile: 16 rows x K (K <= 512 for Q4_K, <= 1024 for IQ2_XXS), fetched whole; IQ2_XXS
// super-scales at +4096.
template <uint32_t TYPE>
__device__ __forceinline__ void issue_down_tile(const uint8_t *mat, uint32_t n_out, uint32_t nb, uint32_t row0, uint8_t *stage, uint64_t *bar,
                                             uint32_t lane) {
    const uint32_t row_bytes = nb * FGeo<TYPE>::BLOCK_BYTES;
    if (lane == 0) {
        fbar_expect(bar, 16 * row_bytes + (TYPE == T_IQ2_XXS ? 16 * nb * 2 : 0));
        fbulk(stage, mat + row0 * row_bytes, 16 * row_bytes, bar);
        if (TYPE == T_IQ2_XXS) fbulk(stage + 4096, mat + n_out * nb * 64u + row0 * nb * 2u, 16 * nb * 2, bar);
    }
}
template <uint32_t TYPE>
__device__ __forceinline__ void consume_down_tile(const uint8_t *stage, uint32_t nb, const uint8_t *lut, const uint8_t *aq_lane,
                                                  const int2 *asum_tok, uint32_t g, uint32_t t, float &f0, float &f1) {
    const uint32_t row_bytes = nb * FGeo<TYPE>::BLOCK_BYTES;
    const uint16_t *d = reinterpret_cast<const uint16_t *>(stage + 4096);
    Halves<TYPE>::run(stage + g * row_bytes, stage + (8 + g) * row_bytes, nb * 2, iq2_swizzle(g, nb), d + g * nb, d + (8 + g) * nb, lut, t,
                      aq_lane, asum_tok, f0, f1);
}

// Two int8 digits per value: v ~ dx * (q1 + q2 / 254), |v| <= 127 dx.  Rounding by the
// 1.5 * 2^23 trick (no conversion instructions): the integer sits in the low mantissa bits, so
// the low byte of the rounded float's bit pattern IS the int8 digit and four of them are packed
// with byte permutes.  `s` accumulates both digit sums: the first in its low half, the second
// in its high half (each below 2^15 in magnitude for a 32-column chunk).
__device__ __forceinline__ void digits4(const float4 v, const float4 c, uint32_t &hi, uint32_t &lo, int &s) {
    const float vv[4] = {v.x, v.y, v.z, v.w};
    const float magic = 12582912.0f;
    uint32_t ra[4], rb[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float r1 = fmaf(vv[j], c.y, magic);
        const float q1 = r1 - magic;
        // second digit clamped to [-127, 127] in the float domain, before the rounding add
        const float r2 = fmaxf(-127.0f, fminf(127.0f, fmaf(-q1, c.x, vv[j]) * c.z)) + magic;
        ra[j] = __float_as_uint(r1); rb[j] = __float_as_uint(r2);
    }
    hi = __byte_perm(__byte_perm(ra[0], ra[1], 0x0040), __byte_perm(ra[2], ra[3], 0x0040), 0x5410);
    lo = __byte_perm(__byte_perm(rb[0], rb[1], 0x0040), __byte_perm(rb[2], rb[3], 0x0040), 0x5410);
    s += __dp4a((int)hi, 0x01010101, 0) + (__dp4a((int)lo, 0x01010101, 0) << 16);
}

// Rows of `k` floats (k % 256 == 0) with known maxima -> digit images, digit sums per 32-column
// chunk and scales.  A warp takes one 256-column segment of one row at a time: two float4 per
// lane, eight consecutive lanes cover one chunk, no index arithmetic beyond the segment's.
// `amax` holds the maxima on entry and the scales (max / 127, or 0 for an unusable row) on
// return; `consts` is scratch, one float4 per row.
// The first `NT` threads of the CTA take part and meet at named barrier `BAR` (0 with NT = FT is the
// CTA barrier).
template <bool GLOBAL, int NT = FT, int BAR = 0>
__device__ __forceinline__ void digitise_rows(const float *src, uint32_t src_pitch, uint32_t rows, uint32_t k, float *amax, uint8_t *dq,
                                           uint32_t dq_pitch, int2 *sums, uint32_t sums_pitch, float4 *consts, uint32_t rotate = 0) {
    auto meet = [] { asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NT) : "memory"); };
#pragma unroll 1
    for (uint32_t r = threadIdx.x; r < rows; r += NT) {
        const float m = amax[r];
        const bool usable = finite_f32(m) && m > 0.0f;
        const float inv = usable ? __fdividef(127.0f, m) : 0.0f;
        consts[r] = make_float4(usable ? m * (1.0f / 127.0f) : 0.0f, inv, 2.0f * inv * 127.0f, 0.0f);
    }
    meet();
    // `rotate`: every CTA reads the same rows from L2; starting each at a different unit keeps them
    // off the same lines at the same time
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, segs = k >> 8, units = rows * segs;
#pragma unroll 1
    for (uint32_t u0 = warp; u0 < units; u0 += NT / 32) {
        const uint32_t u = GLOBAL ? (u0 + rotate * 5u) % units : u0;
        const uint32_t r = u / segs, seg = u - r * segs;
        const float4 *from = reinterpret_cast<const float4 *>(src + (uint64_t)r * src_pitch) + seg * 64u + lane;
        const float4 v0 = GLOBAL ? __ldcg(from) : *from, v1 = GLOBAL ? __ldcg(from + 32) : *(from + 32);
        const float4 c = consts[r];
        uint32_t hi0, lo0, hi1, lo1;
        int s0 = 0, s1 = 0;
        digits4(v0, c, hi0, lo0, s0);
        digits4(v1, c, hi1, lo1, s1);
        uint8_t *out = dq + (2 * r) * dq_pitch + seg * 256u + lane * 4u;
        *reinterpret_cast<uint32_t *>(out) = hi0; *reinterpret_cast<uint32_t *>(out + 128) = hi1;
        *reinterpret_cast<uint32_t *>(out + dq_pitch) = lo0; *reinterpret_cast<uint32_t *>(out + dq_pitch + 128) = lo1;
        for (int o = 1; o < 8; o <<= 1) { s0 += __shfl_xor_sync(0xffffffffu, s0, o); s1 += __shfl_xor_sync(0xffffffffu, s1, o); }
        if ((lane & 7u) == 0) {
            const int a0 = (int)(short)(s0 & 0xffff), a1 = (int)(short)(s1 & 0xffff);
            int2 *to = sums + r * sums_pitch + seg * 8u + (lane >> 3);
            to[0] = make_int2(a0, (s0 - a0) >> 16);
            to[4] = make_int2(a1, (s1 - a1) >> 16);
        }
    }
    meet();
#pragma unroll 1
    for (uint32_t r = threadIdx.x; r < rows; r += NT) amax[r] = consts[r].x;
    meet();
}

__device__ __forceinline__ float fast_sigmoid(float v) {
    const float e = __expf(-fabsf(v));
    return v >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
}

// Softmax, top-k and renormalisation of `tokens` rows of logits in shared memory (zs, FMAXE
// floats per row), CTA-wide; src/qwen4_moe.c:209-247 with its order of operations: ties go to
// the lower id, and with `exact` the exp-sum runs serially over e = 0..E-1 (the reference's
// bits); otherwise it is a warp tree sum.  Returns false (CTA-uniform) when a logit is not
// finite; the first bad row is recorded.
__device__ __forceinline__ bool route_tokens(float *zs, uint32_t E, uint32_t k, int norm, uint32_t T, bool exact, uint32_t *ids_s, float *wts_s,
                                          float *scratch, const unsigned long long *exp_table, uint32_t *flag, uint32_t *status) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid == 0) *flag = 1;
    __syncthreads();
    if (warp < T) {                                                       // row maximum and finiteness
        float m = -CUDART_INF_F;
        bool bad = false;
#pragma unroll 4
        for (uint32_t e = lane; e < E; e += 32) { const float v = zs[warp * FMAXE + e]; bad |= !finite_f32(v); m = fmaxf(m, v); }
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        bad = __any_sync(0xffffffffu, bad);
        if (lane == 0) {
            scratch[warp] = m;
            if (bad) { atomicOr(status, QW4SH_ERR_NONFINITE); atomicMin(status + 1, warp); *flag = 0; }
        }
    }
    __syncthreads();
    if (!*flag) return false;
#pragma unroll 1
    for (uint32_t r = 0; r < T; r++) {                                     // p = expf(z - max)
        const float m = scratch[r];
#pragma unroll 1
        for (uint32_t e = tid; e < E; e += FT) zs[r * FMAXE + e] = expf_libm_table(__fsub_rn(zs[r * FMAXE + e], m), exp_table);
    }
    __syncthreads();
    if (warp < T) {
        const float *p = zs + warp * FMAXE;
        float sum = 0.0f;
        if (exact) {
            if (lane == 0) {                                               // the reference's serial sum
                // 32 values per pass: the loads of the next pass are issued before the 32 dependent adds of this
                // one, and the loop overhead hides under the add chain (a lone warp issues every other cycle)
                uint32_t e = 0;
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = E >= 32 ? *reinterpret_cast<const float4 *>(p + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (; e + 32 <= E; e += 32) {
                    float4 w[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) w[j] = e + 64 <= E ? *reinterpret_cast<const float4 *>(p + e + 32 + 4 * j) : v[j];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        sum = __fadd_rn(sum, v[j].x); sum = __fadd_rn(sum, v[j].y); sum = __fadd_rn(sum, v[j].z); sum = __fadd_rn(sum, v[j].w);
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = w[j];
                }
                for (; e < E; e++) sum = __fadd_rn(sum, p[e]);
            }
            sum = __shfl_sync(0xffffffffu, sum, 0);
        } else {
#pragma unroll 4
            for (uint32_t e = lane; e < E; e += 32) sum += p[e];
            for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (lane == 0) scratch[4 + warp] = sum;
    }
    __syncthreads();
    // the divisions are spread over all warps (the routing warps alone would do sixteen each, one after the other)
#pragma unroll 1
    for (uint32_t e = tid; e < E; e += FT) {                                   // the tokens' divisions of one column are independent: in flight together
#pragma unroll
        for (int r = 0; r < FTOK; r++)
            if ((uint32_t)r < T) zs[r * FMAXE + e] = __fdiv_rn(zs[r * FMAXE + e], scratch[4 + r]);
    }
    __syncthreads();
    if (warp < T) {
        float *p = zs + warp * FMAXE;
        // keys: bits of p / sum (>= 0, so ordered as integers) + 1; a chosen entry becomes -1 (key 0).
        // The row stays in shared memory; every lane keeps the best three keys of its elements (e = lane,
        // lane + 32, ...), so a selection step is two warp reductions, and a lane rescans its elements only
        // when it wins a third time after its last scan.
        uint32_t b1, e1, b2, e2, b3, e3;
        auto scan3 = [&]() {
            b1 = 0; e1 = 0xffffffffu; b2 = 0; e2 = 0xffffffffu; b3 = 0; e3 = 0xffffffffu;
#pragma unroll 4
            for (uint32_t e = lane; e < E; e += 32) {                              // ascending e: the lowest id wins among equals
                const float v = p[e];
                const uint32_t key = v < 0.0f ? 0u : __float_as_uint(v) + 1u;
                if (key > b1) { b3 = b2; e3 = e2; b2 = b1; e2 = e1; b1 = key; e1 = e; }
                else if (key > b2) { b3 = b2; e3 = e2; b2 = key; e2 = e; }
                else if (key > b3) { b3 = key; e3 = e; }
            }
        };
        scan3();
        uint32_t spare = 2;                                                        // valid entries behind the first
        float selected = 0.0f, mine = 0.0f;
#pragma unroll 1
        for (uint32_t slot = 0; slot < k; slot++) {
            const uint32_t top = __reduce_max_sync(0xffffffffu, b1);
            const uint32_t e_win = __reduce_min_sync(0xffffffffu, b1 == top ? e1 : 0xffffffffu);
            const float value = __uint_as_float(top - 1u);
            if (lane == 0) ids_s[warp * k + slot] = e_win;
            if (slot == lane) mine = value;
            if ((e_win & 31u) == lane) {                                           // only this lane's elements changed
                p[e_win] = -1.0f;
                if (spare) { b1 = b2; e1 = e2; b2 = b3; e2 = e3; spare--; }
                else { scan3(); spare = 2; }
            }
            selected = __fadd_rn(selected, value);
        }
        if (lane < k) wts_s[warp * k + lane] = norm ? __fdiv_rn(mine, selected) : mine;
    }
    __syncthreads();
    return true;
}

// ---- the kernel ---------------------------------------------------------------------------------
template <uint32_t RT, uint32_t ST>
__global__ void __launch_bounds__(FT, 1) fused_decode_kernel(const __grid_constant__ FusedArgs args) {
    extern __shared__ __align__(128) uint8_t smem[];
    // The arguments span four cache lines of the constant bank, and a first touch of each line costs a
    // miss that every SM takes at the same moment.  All lines are fetched at once here, into shared
    // memory, and read from there afterwards.
    __shared__ FusedArgs a;
    for (uint32_t i = threadIdx.x; i < sizeof(FusedArgs) / 4; i += FT)
        reinterpret_cast<uint32_t *>(&a)[i] = reinterpret_cast<const uint32_t *>(&args)[i];
    __syncthreads();
    const uint32_t T = a.tokens, H = a.hidden, E = a.experts, k = a.top_k, I = a.inter, IS = a.shared_inter;
    const uint32_t pairs = T * k, rows_c = pairs + T, imax = I > IS ? I : IS;
    constexpr bool LUT = RT == T_IQ2_XXS || ST == T_IQ2_XXS;
    const FPlan p = make_fplan(H, imax, rows_c, a.partial_slices, LUT);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t cta = blockIdx.x, grid = gridDim.x;
    uint64_t *ringbar = reinterpret_cast<uint64_t *>(smem + p.bars);           // [FW][FNS]
    uint64_t *rowbar = ringbar + FW * FNS;                                     // [FRCH]
    uint64_t *lutbar = rowbar + FRCH;
    uint64_t *xbar = lutbar + 1;                                               // x rows (phase A), then the logits (phase B)
    uint32_t *ids_s = reinterpret_cast<uint32_t *>(smem + p.ids);
    float *wts_s = reinterpret_cast<float *>(smem + p.wts);
    float *misc_f = reinterpret_cast<float *>(smem + p.misc);                  // [0..3] x maxima then scales, [4..7] shared logits, [8..15] scratch
    uint32_t *misc_u = reinterpret_cast<uint32_t *>(smem + p.misc) + 16;       // [0] barrier flag, [1] route ok, [2] sources, [4..19] chunk counts
    uint8_t *tokmask = smem + p.tokmask, *slotmap = smem + p.slotmap;
    Src *srcs = reinterpret_cast<Src *>(smem + p.src);
    const uint8_t *lut = smem + p.lut;
    uint8_t *region = smem + p.region;
    uint8_t *xq = region + p.xq;
    int2 *xsum = reinterpret_cast<int2 *>(region + p.xsum);
    uint32_t *amax_g = a.sync + F_SYNC_AMAX;                                   // row maxima of act / shared_act (float bits)
    unsigned long long *clocks = reinterpret_cast<unsigned long long *>(a.sync + F_SYNC_CLOCKS);
    const bool clocked = cta == 0 && tid == 0;
#ifdef QW4_NO_PHASE_CLOCKS
#define CLOCK(i) do { } while (0)
#else
#define CLOCK(i) do { if (clocked) clocks[i] = clock64(); } while (0)
#endif
    CLOCK(0);

    if (tid < FW * FNS + FRCH + 2) {                                           // the barriers lie one after the other: one thread each
        fbar_init(&ringbar[tid], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 8) misc_f[tid] = 0.0f;
    unsigned long long *exp_table = reinterpret_cast<unsigned long long *>(smem + p.misc + 256);
    const unsigned long long exp_entry = tid < 32 ? c_exp2_table[tid] : 0ull;  // a global load: stored to shared memory once x has arrived
    float4 *xconsts = reinterpret_cast<float4 *>(smem + p.misc + 512);
    __syncthreads();
    CLOCK(13);

    // ================================ phase A ================================
    const uint32_t n_rows = cta <= E ? (E - cta) / grid + 1 : 0;              // router rows cta, cta + grid, ... <= E
    uint8_t *xf = region + p.xf;
    uint8_t *rows = region + p.rows;
    const uint32_t chunk_bytes = H;                                            // H * 4 / FRCH
    if (warp == 0) {
        // x first: it is what every warp waits for next
        if (lane == 30) fbar_expect(xbar, T * H * 4u);
        if (lane < FRCH) fbar_expect(&rowbar[lane], n_rows * chunk_bytes);
        __syncwarp();
        if (lane < T) fbulk(xf + lane * p.xf_pitch, a.x + (uint64_t)lane * H, H * 4u, xbar);
        if (LUT && lane == 31) {
            fbar_expect(lutbar, F_LUT_BYTES);
            fbulk(smem + p.lut, a.lut, F_LUT_BYTES, lutbar);
        }
    } else if (warp >= 2 && warp < 2 + n_rows && lane < FRCH) {                // router row warp - 2: one request per chunk and lane.  (Requests cost
        const uint32_t j = warp - 2, c = lane, r = cta + j * grid;             // the issuing warp some 50 cycles each, so they are dealt out; a copy
        const uint8_t *src = r < E ? a.w[0].data + (uint64_t)r * a.w[0].row_bytes : a.w[7].data;      // may land before warp 0's expect.)
        fbulk(rows + j * p.row_pitch + c * chunk_bytes, src + c * chunk_bytes, chunk_bytes, &rowbar[c]);
    } else if (warp == 1 && lane < 3) {                                        // the shared expert's tensors -> L2: one request per tensor
        const uint32_t m = 4 + lane;                                            // (a warp that issues dozens of them holds the CTA barrier up)
        const uint32_t bytes = (uint32_t)a.w[m].expert_bytes & ~15u;            // shared tensors are far below 4 GB
        const uint32_t sub = ((bytes / grid) + 16u) & ~15u;
        const uint32_t from = cta * sub;
        if (from < bytes) fprefetch_l2(a.w[m].data + from, from + sub <= bytes ? sub : bytes - from);
    }
    // x -> shared memory (float, one bulk copy per row) with the row maxima, then digits; token rows beyond T stay zero
    bool alive = fbar_wait(xbar, 0, a.status);
    if (tid < 32) exp_table[tid] = exp_entry;
    CLOCK(14);
    {
        float m[FTOK] = {0.f, 0.f, 0.f, 0.f};
        if (alive) {
#pragma unroll 1
            for (uint32_t c4 = tid; c4 < (H >> 2); c4 += FT) {                  // the rows' loads of one column are in flight together
#pragma unroll
                for (int q = 0; q < FTOK; q++) {
                    if ((uint32_t)q < T) {
                        const float4 v = *reinterpret_cast<const float4 *>(xf + q * p.xf_pitch + c4 * 16);
                        m[q] = fmaxf(m[q], fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < FTOK; q++) {
            float v = m[q];
            for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0 && v > 0.0f) atomicMax(reinterpret_cast<uint32_t *>(misc_f) + q, __float_as_uint(v));
        }
        CLOCK(15);
#pragma unroll 1
        for (uint32_t i = tid; i < (FTOK - T) * 2 * (p.kp >> 4); i += FT)       // digit rows of absent tokens
            reinterpret_cast<uint4 *>(xq + 2 * T * p.kp)[i] = make_uint4(0, 0, 0, 0);
#pragma unroll 1
        for (uint32_t i = tid; i < (FTOK - T) * (H >> 5); i += FT) xsum[T * (H >> 5) + i] = make_int2(0, 0);
    }
    __syncthreads();
    CLOCK(1);
    if (a.router_mode != 0) digitise_rows<false>(reinterpret_cast<const float *>(xf), p.xf_pitch >> 2, T, H, misc_f, xq, p.kp, xsum, H >> 5, xconsts);
    CLOCK(2);
    // router rows
    if (a.router_mode == 0) {
        // Exact order: every (row, token) logit is one chain of K separately rounded adds, and a lone
        // warp issues too slowly to also load and multiply.  So the other warps write the products
        // (the same separately rounded multiplies) chunk by chunk into a two-buffer ring, and the
        // last warp only loads and adds: lane = chain.  Named barriers 2/3 say "buffer filled",
        // 4/5 "buffer drained".
        float *prod = reinterpret_cast<float *>(region + p.prod);              // [2][16 chains][chunk + 4]
        const uint32_t chunk = H / FRCH, ppitch = chunk + 4, chains = n_rows * T;
        uint8_t *chain_map = smem + p.misc + 640;                              // chain -> router row of this CTA | token << 4
        if (tid < chains) chain_map[tid] = (uint8_t)((tid / T) | ((tid % T) << 4));
        __syncthreads();
        if (warp == FW - 1) {
            float sum = 0.0f;
#pragma unroll 1
            for (uint32_t c = 0; c < FRCH; c++) {
                asm volatile("bar.sync %0, %1;" ::"r"(2 + (c & 1u)), "n"(FT) : "memory");
                if (lane < chains) {
                    const float4 *pv = reinterpret_cast<const float4 *>(prod + ((c & 1u) * 16 + lane) * ppitch);
#pragma unroll 4
                    for (uint32_t i = 0; i < chunk / 4; i++) {
                        const float4 q = pv[i];
                        sum = __fadd_rn(sum, q.x); sum = __fadd_rn(sum, q.y); sum = __fadd_rn(sum, q.z); sum = __fadd_rn(sum, q.w);
                    }
                }
                if (c + 2 < FRCH) asm volatile("bar.arrive %0, %1;" ::"r"(4 + (c & 1u)), "n"(FT) : "memory");
            }
            if (lane < chains) {
                const uint32_t j = lane / T, tok = lane % T, r = cta + j * grid;
                if (!finite_f32(sum)) { atomicOr(a.status, QW4SH_ERR_NONFINITE); atomicMin(a.status + 1, tok); }
                if (r < E) a.logits[(uint64_t)tok * E + r] = sum; else a.shared_logit[tok] = sum;
            }
        } else {
#pragma unroll 1
            for (uint32_t c = 0; c < FRCH; c++) {
                if (alive) alive = fbar_wait(&rowbar[c], 0, a.status);           // on a failed wait the products are garbage, the flag is set
                if (c >= 2) asm volatile("bar.sync %0, %1;" ::"r"(4 + (c & 1u)), "n"(FT) : "memory");
                // one unit = 32 float4 of one chain: no index arithmetic beyond a table look-up per unit
#pragma unroll 1
                for (uint32_t u = warp; u < chains * (chunk / 128); u += FW - 1) {
                    const uint32_t ch = u / (chunk / 128), q4 = (u % (chunk / 128)) * 32 + lane;
                    const uint32_t jt = chain_map[ch], j = jt & 15u, tok = jt >> 4;
                    const float4 w4 = *reinterpret_cast<const float4 *>(rows + j * p.row_pitch + c * chunk_bytes + q4 * 16);
                    const float4 x4 = *reinterpret_cast<const float4 *>(xf + tok * p.xf_pitch + c * chunk_bytes + q4 * 16);
                    *reinterpret_cast<float4 *>(prod + ((c & 1u) * 16 + ch) * ppitch + q4 * 4) =
                        make_float4(__fmul_rn(w4.x, x4.x), __fmul_rn(w4.y, x4.y), __fmul_rn(w4.z, x4.z), __fmul_rn(w4.w, x4.w));
                }
                asm volatile("bar.arrive %0, %1;" ::"r"(2 + (c & 1u)), "n"(FT) : "memory");
                // both product buffers are full and the chain warp is busy with them: the digit image of x is
                // built here, under the chain
                if (c == 1) digitise_rows<false, FT - 32, 6>(reinterpret_cast<const float *>(xf), p.xf_pitch >> 2, T, H, misc_f, xq, p.kp, xsum,
                                                              H >> 5, xconsts);
            }
        }
    } else {
#pragma unroll 1
        for (uint32_t c = 0; c < FRCH && alive; c++) alive = fbar_wait(&rowbar[c], 0, a.status);
#pragma unroll 1
        for (uint32_t dot = warp; dot < n_rows * T && alive; dot += FW) {
            const uint32_t j = dot / T, tok = dot % T;
            const float4 *wv = reinterpret_cast<const float4 *>(rows + j * p.row_pitch);
            const float4 *xv = reinterpret_cast<const float4 *>(xf + tok * p.xf_pitch);
            float acc = 0.0f;
#pragma unroll 1
            for (uint32_t i = lane; i < (H >> 2); i += 32) {
                const float4 w4 = wv[i], x4 = xv[i];
                acc = fmaf(w4.x, x4.x, fmaf(w4.y, x4.y, fmaf(w4.z, x4.z, fmaf(w4.w, x4.w, acc))));
            }
            for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) {
                const uint32_t r = cta + j * grid;
                if (!finite_f32(acc)) { atomicOr(a.status, QW4SH_ERR_NONFINITE); atomicMin(a.status + 1, tok); }
                if (r < E) a.logits[(uint64_t)tok * E + r] = acc; else a.shared_logit[tok] = acc;
            }
        }
    }
    alive = __all_sync(0xffffffffu, alive);
    CLOCK(3);
    if (!grid_barrier(a.sync + 0, grid, a.status, misc_u)) return;
    CLOCK(4);

    // ================================ phase B ================================
    float *zs = reinterpret_cast<float *>(region + p.zs);
    const bool bulk_logits = (E & 3u) == 0;                                   // whole 16-byte pieces: one bulk copy per token row
    if (bulk_logits) {
        if (warp == 0 && alive) {
            asm volatile("fence.proxy.async;" ::: "memory");                      // generic-proxy writes (the logits; phase A's use of this memory) before the copy
            if (lane == 0) fbar_expect(xbar, T * E * 4u);
            __syncwarp();
            if (lane < T) fbulk(zs + lane * FMAXE, a.logits + (uint64_t)lane * E, E * 4u, xbar);
        }
    } else {
#pragma unroll 1
        for (uint32_t r = 0; r < T; r++)
#pragma unroll 1
            for (uint32_t e = tid; e < E; e += FT) zs[r * FMAXE + e] = __ldcg(a.logits + (uint64_t)r * E + e);
    }
    if (tid < T) misc_f[4 + tid] = __ldcg(a.shared_logit + tid);
#pragma unroll 1
    for (uint32_t i = tid; i < FMAXE; i += FT) tokmask[i] = 0;
    if (bulk_logits && alive) alive = fbar_wait(xbar, 1, a.status);            // second use of this barrier: phase parity 1
    __syncthreads();
    CLOCK(5);
    const bool routed_ok = route_tokens(zs, E, k, a.norm, T, a.router_mode == 0, ids_s, wts_s, misc_f + 8, exp_table, misc_u + 1, a.status);
    CLOCK(6);
    if (routed_ok) {
        if (tid < pairs) {
            const uint32_t e = ids_s[tid], tok = tid / k;
            atomicOr(reinterpret_cast<uint32_t *>(tokmask) + (e >> 2), (1u << tok) << (8 * (e & 3u)));
            slotmap[e * 4 + tok] = (uint8_t)(tid % k);
            if (cta == 0) {
                a.ids[tid] = e; a.weights[tid] = wts_s[tid];
                if (a.ids_out) a.ids_out[tid] = e;
                if (a.weights_out) a.weights_out[tid] = wts_s[tid];
            }
        }
        __syncthreads();
        // distinct experts in ascending order behind the shared expert (source 0)
#pragma unroll 1
        for (uint32_t c = warp; c < (E + 31) / 32; c += FW) {
            const uint32_t e = c * 32 + lane;
            const uint32_t any = __ballot_sync(0xffffffffu, e < E && tokmask[e] != 0);
            if (lane == 0) misc_u[4 + c] = __popc(any);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t running = 1;
#pragma unroll 1
            for (uint32_t c = 0; c < (E + 31) / 32; c++) { const uint32_t n = misc_u[4 + c]; misc_u[4 + c] = running; running += n; }
            misc_u[2] = running;
            Src s; s.expert = 0xffffu; s.mask = (uint8_t)((1u << T) - 1u); s.shared = 1; s.slots = 0;
            srcs[0] = s;
        }
        __syncthreads();
#pragma unroll 1
        for (uint32_t c = warp; c < (E + 31) / 32; c += FW) {
            const uint32_t e = c * 32 + lane;
            const bool has = e < E && tokmask[e] != 0;
            const uint32_t any = __ballot_sync(0xffffffffu, has);
            if (has) {
                Src s; s.expert = (uint16_t)e; s.mask = tokmask[e]; s.shared = 0;
                s.slots = *reinterpret_cast<const uint32_t *>(slotmap + e * 4);
                srcs[misc_u[4 + c] + __popc(any & ((1u << lane) - 1u))] = s;
            }
        }
        __syncthreads();
    }
    const uint32_t n_src = routed_ok ? misc_u[2] : 0;
    CLOCK(7);
    uint32_t ring_count = 0;                                                   // slices this warp has pushed through its ring
    uint64_t *bar = ringbar + warp * FNS;
    if (routed_ok) {
        // gate/up units: shared expert first, then the routed experts; whole units per CTA
        const uint32_t us = IS >> 3, ur = I >> 3, total = us + (n_src - 1) * ur;
        const uint32_t u0 = total * cta / grid, u1 = total * (cta + 1) / grid;            // total <= 65 * 128: no overflow
        const uint32_t n_shu = u0 < us ? min(us, u1) - u0 : 0;                 // shared units of this CTA come first
        const uint32_t nbh = H >> 8;
        const uint32_t spu_s = nbh / FGeo<ST>::SLICE_BLOCKS, spu_r = nbh / FGeo<RT>::SLICE_BLOCKS;
        const uint32_t slices = min(n_shu * spu_s + (u1 - u0 - n_shu) * spu_r, a.partial_slices);
        const uint32_t mine = slices > warp ? (slices - 1 - warp) / FW + 1 : 0;
        uint8_t *ring = region + p.ring + warp * FNS * FSTAGE;
        float2 *partial = reinterpret_cast<float2 *>(region + p.partial);
        if (LUT && alive) alive = fbar_wait(lutbar, 0, a.status);
        alive = __all_sync(0xffffffffu, alive);
        auto locate = [&](uint32_t n, uint32_t &ul, uint32_t &s, bool &sh) {   // CTA slice n -> local unit, slice, kind
            if (n < n_shu * spu_s) { ul = n / spu_s; s = n % spu_s; sh = true; }
            else { const uint32_t m = n - n_shu * spu_s; ul = n_shu + m / spu_r; s = m % spu_r; sh = false; }
        };
        auto issue = [&](uint32_t i) {
            uint32_t ul, s; bool sh;
            locate(warp + i * FW, ul, s, sh);
            const uint32_t u = u0 + ul;
            uint8_t *stage = ring + (i % FNS) * FSTAGE;
            if (sh) issue_unit_slice<ST>(a.w[4].data, a.w[5].data, IS, nbh, u * 8, s, stage, &bar[i % FNS], lane);
            else {
                const uint32_t v = u - us, e = srcs[1 + v / ur].expert;
                issue_unit_slice<RT>(a.w[1].data + (uint64_t)e * a.w[1].expert_bytes, a.w[2].data + (uint64_t)e * a.w[2].expert_bytes, I, nbh,
                                     (v % ur) * 8, s, stage, &bar[i % FNS], lane);
            }
        };
        if (alive) for (uint32_t i = 0; i < FNS && i < mine; i++) issue(i);
        // down tiles of this CTA's columns -> L2, ahead of phase C
#pragma unroll 1
        for (uint32_t tile = cta; tile < (H >> 4); tile += grid)
            for (uint32_t j = warp * 4 + lane; lane < 4 && j < n_src; j += FW * 4) {      // a few requests per warp: none of them falls behind
                const Src s = srcs[j];
                const uint32_t rb = s.shared ? (IS >> 8) * (ST == T_Q4_K ? 144u : 64u) : (I >> 8) * (RT == T_Q4_K ? 144u : 64u);
                const uint8_t *mat = s.shared ? a.w[6].data : a.w[3].data + (uint64_t)s.expert * a.w[3].expert_bytes;
                fprefetch_l2(mat + tile * 16 * rb, 16 * rb);
            }
        const uint8_t *xq_lane = xq + g * p.kp + 8 * t;
        const int2 *xsum_tok = xsum + t * (H >> 5);
#pragma unroll 1
        for (uint32_t i = 0; i < mine; i++) {
            uint32_t ul, s; bool sh;
            locate(warp + i * FW, ul, s, sh);
            if (alive) alive = fbar_wait(&bar[i % FNS], (i / FNS) & 1u, a.status);
            alive = __all_sync(0xffffffffu, alive);
            const uint8_t *stage = ring + (i % FNS) * FSTAGE;
            float f0 = 0.0f, f1 = 0.0f;
            if (alive) {
                if (sh) consume_unit_slice<ST>(stage, nbh, s, lut, xq_lane, xsum_tok, g, t, f0, f1);
                else consume_unit_slice<RT>(stage, nbh, s, lut, xq_lane, xsum_tok, g, t, f0, f1);
            }
            partial[(warp + i * FW) * 32 + lane] = make_float2(f0, f1);
            __syncwarp();
            fproxy_fence();
            if (alive && i + FNS < mine) issue(i + FNS);
        }
        ring_count = alive ? mine : 0;
        CLOCK(8);
        __syncthreads();
        // units: slices added in order, SwiGLU, store, row maxima
#pragma unroll 1
        for (uint32_t ul = warp; ul < u1 - u0; ul += FW) {
            const bool sh = ul < n_shu;
            const uint32_t spu = sh ? spu_s : spu_r;
            const uint32_t n0 = sh ? ul * spu_s : n_shu * spu_s + (ul - n_shu) * spu_r;
            if (n0 + spu > slices) break;                                      // beyond the partial buffer (never for supported shapes)
            float f0 = 0.0f, f1 = 0.0f;
#pragma unroll 1
            for (uint32_t s = 0; s < spu; s++) { const float2 v = partial[(n0 + s) * 32 + lane]; f0 += v.x; f1 += v.y; }
            const uint32_t u = u0 + ul;
            float v = 0.0f;
            uint32_t row = 0;
            bool live = false;
            if (t < T) {
                const float dx = misc_f[t];
                const float gate = f0 * dx, upv = f1 * dx;
                v = gate * fast_sigmoid(gate) * upv;
                if (sh) { live = true; row = pairs + t; a.shared_act[(uint64_t)t * IS + u * 8 + g] = v; }
                else {
                    const uint32_t vu = u - us;
                    const Src sr = srcs[1 + vu / ur];
                    if ((sr.mask >> t) & 1u) { live = true; row = t * k + sr.slot(t); a.act[(uint64_t)row * I + (vu % ur) * 8 + g] = v; }
                }
                if (live && !finite_f32(v)) atomicOr(a.status, QW4SH_ERR_NONFINITE);
            }
            float m = live ? fabsf(v) : 0.0f;                                  // maximum over the unit's eight rows (lanes of equal t)
            for (int o = 4; o < 32; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (live && g == 0 && m > 0.0f) atomicMax(amax_g + row, __float_as_uint(m));
        }
    }
    CLOCK(9);
    if (!grid_barrier(a.sync + 1, grid, a.status, misc_u)) return;
    CLOCK(10);

    // ================================ phase C ================================
    if (routed_ok && cta < (H >> 4)) {
        uint8_t *aq = region + p.aq;
        int2 *asum = reinterpret_cast<int2 *>(region + p.asum);
        float *ascale = reinterpret_cast<float *>(region + p.ascale);
        uint8_t *tiles = region + p.tiles + warp * FNS * FSTAGE;
        float2 *cpartial = reinterpret_cast<float2 *>(region + p.cpartial);
        const uint32_t my_src = n_src > warp ? (n_src - 1 - warp) / FW + 1 : 0;
        const uint32_t n_tiles = ((H >> 4) - cta + grid - 1) / grid;
        const uint32_t steps = my_src * n_tiles;
        auto issue = [&](uint32_t n) {                                         // the ring barriers go on counting where phase B left them
            const uint32_t tile = cta + (n / my_src) * grid, j = warp + (n % my_src) * FW;
            const Src s = srcs[j];
            const uint32_t at = ring_count + n;
            uint8_t *stage = tiles + (at % FNS) * FSTAGE;
            if (s.shared) issue_down_tile<ST>(a.w[6].data, H, IS >> 8, tile * 16, stage, &bar[at % FNS], lane);
            else issue_down_tile<RT>(a.w[3].data + (uint64_t)s.expert * a.w[3].expert_bytes, H, I >> 8, tile * 16, stage, &bar[at % FNS], lane);
        };
        // digit images of the activation rows: pairs first, then the shared expert's rows
#pragma unroll 1
        for (uint32_t r = tid; r < rows_c; r += FT) ascale[r] = __uint_as_float(__ldcg(amax_g + r));
        float4 *aconsts = reinterpret_cast<float4 *>(region + p.aconst);
        // The rows were written by other CTAs a moment ago and every CTA needs all of them.  Read with ordinary
        // loads they cost a chain of L2 round trips; when they fit the (still idle) tile ring they come in with
        // one bulk copy per row instead and are digitised out of shared memory.
        const bool staged = rows_c * imax * 4u <= FW * FNS * FSTAGE && ((I | IS) & 3u) == 0;
        if (staged) {
            float *stage = reinterpret_cast<float *>(region + p.tiles);
            bool ok = __syncthreads_and(alive);                                    // CTA-uniform from here on: the digitiser meets at CTA barriers
            if (ok) {
                if (tid == 0) fbar_expect(&rowbar[0], (pairs * I + T * IS) * 4u);
                if (lane < 4) {                                                   // four requests per warp
                    asm volatile("fence.proxy.async;" ::: "memory");              // the rows were written through the generic proxy
#pragma unroll 1
                    for (uint32_t r = warp * 4 + lane; r < rows_c; r += FW * 4) {
                        if (r < pairs) fbulk(stage + r * I, a.act + (uint64_t)r * I, I * 4u, &rowbar[0]);
                        else fbulk(stage + pairs * I + (r - pairs) * IS, a.shared_act + (uint64_t)(r - pairs) * IS, IS * 4u, &rowbar[0]);
                    }
                }
                ok = __syncthreads_and(fbar_wait(&rowbar[0], 1, a.status));         // second use of this barrier: phase parity 1
            }
            if (ok) {
                if (I == IS) digitise_rows<false>(stage, I, rows_c, I, ascale, aq, p.ap, asum, imax >> 5, aconsts);
                else {
                    digitise_rows<false>(stage, I, pairs, I, ascale, aq, p.ap, asum, imax >> 5, aconsts);
                    digitise_rows<false>(stage + pairs * I, IS, T, IS, ascale + pairs, aq + 2 * pairs * p.ap, p.ap, asum + pairs * (imax >> 5),
                                            imax >> 5, aconsts + pairs);
                }
            }
            alive = ok;
            fproxy_fence();                                                        // the ring goes back to the bulk copies
            if (alive) for (uint32_t n = 0; n < FNS && n < steps; n++) issue(n);
        } else {
            fproxy_fence();
            if (alive) for (uint32_t n = 0; n < FNS && n < steps; n++) issue(n);
            __syncthreads();
            digitise_rows<true>(a.act, I, pairs, I, ascale, aq, p.ap, asum, imax >> 5, aconsts, cta);
            digitise_rows<true>(a.shared_act, IS, T, IS, ascale + pairs, aq + 2 * pairs * p.ap, p.ap, asum + pairs * (imax >> 5), imax >> 5,
                                   aconsts + pairs, cta);
        }
        CLOCK(11);
        uint32_t n = 0;
#pragma unroll 1
        for (uint32_t ti = 0; ti < n_tiles; ti++) {
            const uint32_t tile = cta + ti * grid;
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 1
            for (uint32_t si = 0; si < my_src; si++, n++) {
                const Src s = srcs[warp + si * FW];
                const uint32_t tokg = g >> 1;
                const uint32_t row_g = s.shared ? pairs + (tokg < T ? tokg : 0) : (((s.mask >> tokg) & 1u) ? tokg * k + s.slot(tokg) : 0);
                const bool live_t = t < T && ((s.mask >> t) & 1u);
                const uint32_t row_t = s.shared ? pairs + (t < T ? t : 0) : (live_t ? t * k + s.slot(t) : 0);
                const uint8_t *aq_lane = aq + (2 * row_g + (g & 1u)) * p.ap + 8 * t;
                const int2 *asum_tok = asum + row_t * (imax >> 5);
                const uint32_t at = ring_count + n;
                if (alive) alive = fbar_wait(&bar[at % FNS], (at / FNS) & 1u, a.status);
                alive = __all_sync(0xffffffffu, alive);
                const uint8_t *stage = tiles + (at % FNS) * FSTAGE;
                float f0 = 0.0f, f1 = 0.0f;
                if (alive) {
                    if (s.shared) consume_down_tile<ST>(stage, IS >> 8, lut, aq_lane, asum_tok, g, t, f0, f1);
                    else consume_down_tile<RT>(stage, I >> 8, lut, aq_lane, asum_tok, g, t, f0, f1);
                }
                __syncwarp();
                fproxy_fence();
                if (alive && n + FNS < steps) issue(n + FNS);
                if (live_t) {
                    const float coef = (s.shared ? fast_sigmoid(misc_f[4 + t]) : wts_s[t * k + s.slot(t)]) * ascale[row_t];
                    acc0 = fmaf(coef, f0, acc0); acc1 = fmaf(coef, f1, acc1);
                }
            }
            cpartial[warp * 32 + lane] = make_float2(acc0, acc1);
            __syncthreads();
            if (tid < 64) {                                                    // rows g (threads 0-31) and g + 8 (32-63), warps added in order
                const uint32_t l = tid & 31u, gg = l >> 2, tt = l & 3u, hi = tid >> 5;
                float sum = 0.0f;
#pragma unroll 1
                for (uint32_t w = 0; w < FW; w++) {
                    const float2 v = cpartial[w * 32 + l];
                    sum += hi ? v.y : v.x;
                }
                if (tt < T) {
                    if (!finite_f32(sum)) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.y[(uint64_t)tt * H + tile * 16 + hi * 8 + gg] = sum;
                }
            }
            __syncthreads();
        }
    }
    CLOCK(12);
    // the CTA that leaves last clears the counters and the row maxima for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        misc_u[0] = atomicAdd(a.sync + 2, 1u) == grid - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (misc_u[0]) {
#pragma unroll 1
        for (uint32_t r = tid; r < rows_c; r += FT) amax_g[r] = 0;
        if (tid == 0) { a.sync[0] = 0; a.sync[1] = 0; a.sync[2] = 0; }
        __threadfence();
    }
#undef CLOCK
}

}  // namespace qw4

using namespace qw4;

extern "C" int qw4sh_note_launch(const char *name);
extern "C" const uint8_t *qw4sh_lut_image(void);

static DevTensor fdev(const QW4ShTensor &s) {
    DevTensor t;
    t.data = s.data; t.type = s.type; t.k_storage = s.k_storage; t.k_logical = s.k_logical;
    t.n_out = s.n_out; t.n_experts = s.n_experts; t.row_bytes = s.row_bytes; t.expert_bytes = s.expert_bytes;
    return t;
}

static int g_fused_mode = -1;                          // -1 automatic, 0 never
extern "C" void qw4sh_set_fused_decode(int mode) { g_fused_mode = mode; }

static bool fused_type(uint32_t type) { return type == T_Q4_K || type == T_IQ2_XXS; }
static uint32_t slice_blocks(uint32_t type) { return type == T_Q4_K ? FGeo<T_Q4_K>::SLICE_BLOCKS : FGeo<T_IQ2_XXS>::SLICE_BLOCKS; }

// Most slices one CTA can get: its share of the units (whole units, the shared expert's first),
// each cut into its format's number of slices.
static uint32_t partial_capacity(const QW4ShLayer *l, size_t tokens, int grid) {
    const uint32_t nbh = l->hidden >> 8, spu_s = nbh / slice_blocks(l->w[4].type), spu_r = nbh / slice_blocks(l->w[1].type);
    const uint32_t us = l->shared_inter >> 3, ur = l->inter >> 3;
    const uint64_t total = us + (uint64_t)tokens * l->top_k * ur;
    const uint32_t per_cta = (uint32_t)((total + grid - 1) / grid) + 1;
    return per_cta * (spu_s > spu_r ? spu_s : spu_r);
}

static FPlan plan_for(const QW4ShLayer *l, size_t tokens, int grid) {
    const uint32_t imax = l->inter > l->shared_inter ? l->inter : l->shared_inter;
    const bool lut = l->w[1].type == T_IQ2_XXS || l->w[4].type == T_IQ2_XXS;
    return make_fplan(l->hidden, imax, (uint32_t)tokens * l->top_k + (uint32_t)tokens, partial_capacity(l, tokens, grid), lut);
}

// Whether the one-kernel decode path covers this layer and batch.
extern "C" int qw4sh_fused_supported(const QW4ShLayer *l, size_t tokens, const float *x, const float *y, int grid) {
    if (g_fused_mode == 0) return 0;
    if (!tokens || tokens > FTOK || l->top_k > FMAXK || l->experts > FMAXE || l->top_k > l->experts) return 0;
    const uint32_t H = l->hidden, I = l->inter, IS = l->shared_inter;
    if (H % 1024 || H > 4096 || I % 256 || IS % 256 || !I || !IS) return 0;
    if (((uintptr_t)x | (uintptr_t)y) & 15u) return 0;
    if (l->w[0].type != T_F32 || l->w[7].type != T_F32) return 0;
    const uint32_t rt = l->w[1].type, st = l->w[4].type;
    if (!fused_type(rt) || !fused_type(st)) return 0;
    if (l->w[2].type != rt || l->w[3].type != rt || l->w[5].type != st || l->w[6].type != st) return 0;
    for (int i = 1; i <= 6; i++) if (l->w[i].k_logical != l->w[i].k_storage) return 0;
    // a down tile (16 rows) must fit one ring stage
    if (rt == T_Q4_K ? I > 512 : I > 1024) return 0;
    if (st == T_Q4_K ? IS > 512 : IS > 1024) return 0;
    if (grid < 1 || (uint32_t)grid * FRMAX < l->experts + 1) return 0;
    if (tokens * l->top_k + tokens > 192) return 0;                      // row maxima live in the sync array
    if (plan_for(l, tokens, grid).total > 227u * 1024u) return 0;
    return 1;
}

template <uint32_t RT, uint32_t ST>
static int launch_fused(const FusedArgs &a, uint32_t smem, int grid, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(fused_decode_kernel<RT, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(FT); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, fused_decode_kernel<RT, ST>, a);
    if (e != cudaSuccess) return (int)e;
    return qw4sh_note_launch("fused_decode_kernel");
}

extern "C" int qw4sh_fused_decode(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens,
                                  uint32_t *ids_out, float *weights_out, int router_mode, int sm_count) {
    FusedArgs a;
    for (int i = 0; i < 8; i++) a.w[i] = fdev(layer->w[i]);
    a.x = x; a.y = y;
    a.tokens = (uint32_t)tokens; a.hidden = layer->hidden; a.experts = layer->experts; a.top_k = layer->top_k;
    a.inter = layer->inter; a.shared_inter = layer->shared_inter; a.norm = layer->norm; a.router_mode = router_mode;
    a.logits = work->logits; a.shared_logit = work->shared_logit; a.ids = work->ids; a.weights = work->weights;
    a.act = work->act; a.shared_act = work->shared_act; a.ids_out = ids_out; a.weights_out = weights_out;
    a.sync = work->sync; a.status = work->status;
    const uint32_t rt = layer->w[1].type, st = layer->w[4].type;
    const bool lut = rt == T_IQ2_XXS || st == T_IQ2_XXS;
    a.lut = lut ? qw4sh_lut_image() : nullptr;
    if (lut && !a.lut) return -3;
    a.partial_slices = partial_capacity(layer, tokens, sm_count);
    const FPlan p = plan_for(layer, tokens, sm_count);
    if (p.total > 227u * 1024u) return -4;
    cudaStream_t s = (cudaStream_t)work->stream;
    if (rt == T_Q4_K) return st == T_Q4_K ? launch_fused<T_Q4_K, T_Q4_K>(a, p.total, sm_count, s) : launch_fused<T_Q4_K, T_IQ2_XXS>(a, p.total, sm_count, s);
    return st == T_Q4_K ? launch_fused<T_IQ2_XXS, T_Q4_K>(a, p.total, sm_count, s) : launch_fused<T_IQ2_XXS, T_IQ2_XXS>(a, p.total, sm_count, s);
}
