// The whole MoE layer for a decode step of up to four tokens as ONE persistent kernel (sm_100a).
//
// One CTA per SM, all resident at once; picoforge src/qwen4_moe.c:334-382 is the CPU statement of
// the sequence.  The CTAs have two roles.
//
// CHAIN CTAs (the first NC) own the reference's router arithmetic: every logit is one chain of K
// separately rounded multiply-adds in ascending k (src/qwen4_packed.c:164-173), 32 router rows
// per CTA, one warp per token, lane = row, the rows streamed through a swizzled cp.async ring by
// the CTA's other warps.  A chain is 2048 dependent adds, about 9 k cycles whatever else happens,
// so it is kept OFF the critical path: when all chains are done, chain CTA t routes token t
// (libm-exact softmax, serial exp-sum, top-k, renormalisation: src/qwen4_moe.c:209-247) and
// publishes ids and weights.
//
// STREAMING CTAs (all others) do not wait for that.  They compute tree-summed logits of their 3-4
// router rows at once (phase A), exchange them through the first grid-wide barrier, take the
// top-k SET of every token from those logits (a speculation: the tree sums differ from the chains
// in the last bits, which matters only for a near-tie at the k-th place) and stream the gate/up
// rows of the experts in that set (phase B).  At the second barrier they also wait for the chain
// CTAs' routes and compare: if a token's exact expert set differs from the speculated one, phase B
// runs again with the exact ids, so ids and weights are always the reference's bits.  Phase C
// (down projection, weighted combine, sigmoid-gated shared expert) uses the exact weights.
//
//   A  x -> shared memory, int8 digit pairs of x, tree-summed logits of rows sc, sc + NS, ...
//   B  work unit = 8 gate rows + the same 8 up rows of one expert (gate in MMA rows 0-7, up in
//      8-15); a unit is cut into slices of 512 columns dealt to the CTA's warps, each warp fetching
//      slices into its own ring (Q4_K: one 3-D tensor-map request per matrix; IQ2_XXS: one bulk copy
//      of a contiguous span of its expanded image) and feeding int8 tensor-core MMAs with the codes.
//      Units come in granules of four (32 activation columns): the warp that sums a granule's
//      slices applies SwiGLU and writes the activation as int8 digit pairs with ONE SCALE PER
//      32-COLUMN CHUNK, so that no row maximum has to cross the grid and phase C starts with a
//      bulk copy of ready-made digits.
//   C  streaming CTA sc owns 16 columns of y: its warps split the sources (shared expert +
//      distinct routed experts), each runs the 16 x K down tile on the tensor cores against the
//      digits of the pair's activation, scales by the route weight (or the sigmoid gate), and the
//      partial sums are added in warp order: y is deterministic.
//
// The kernel is launched as a normal grid of one CTA per SM with programmatic stream
// serialisation: the next layer's launch may begin while this one drains, and everything that
// touches memory another launch writes comes after griddepcontrol.wait.  All CTAs are resident
// together because each needs more than half of an SM's shared memory and the grid is the SM
// count; every wait (mbarrier, counter) is bounded: after about a second the kernel records
// QW4SH_ERR_STATE and leaves.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

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
constexpr int FRMAX = 4;                        // router rows per streaming CTA
constexpr int FNS = 2;                          // ring stages per warp, gate/up phase (three stages fit and were measured: no faster)
constexpr int FNC = 2;                          // ring stages per warp, down phase
constexpr uint32_t FSTAGE = 4608;               // bytes per ring stage: 16 rows x 288 bytes (512 columns of either format)
constexpr uint32_t FZP = FMAXE + 4;             // pitch of a logit row in shared memory (floats)
constexpr int CROWS = 32;                       // router rows per chain CTA (lane = row).  64 rows (two chain warps per token, nine
                                                // chain CTAs) evened out the streaming CTAs' shares but ran the chains at 42 k cycles
                                                // instead of 25 k, and the step at 44.4 us instead of 42.0
constexpr int CSTG = 16;                        // chunks in flight in a chain CTA
constexpr int CCH = 64;                         // columns per chunk: 256 bytes per row
// words of the sync array
enum : uint32_t { S_FAST = 0, S_CHAIN = 1, S_ROUTED = 2, S_ACT0 = 3, S_ACT1 = 4, S_EXITS = 5, S_ROUTE_FAIL = 6, S_CLOCKS = 8, S_REPAIRS = 48, S_MARKS = 256 };

struct FusedArgs {
    DevTensor w[8];                             // router, gate, up, down, sgate, sup, sdown, srouter
    const float *x;
    float *y;
    uint32_t tokens, hidden, experts, top_k, inter, shared_inter;
    int norm, router_mode;                      // 0 exact, 1 fast, 2 exact with a wrong speculation forced (test aid)
    float *logits, *shared_logit;               // [T, E], [T]: the logits the routes were made from
    float *logits_fast;                         // [T, fast_pitch]: tree sums, the shared router's at column E
    uint32_t fast_pitch;
    uint32_t *ids;                              // [T, k]
    float *weights;                             // [T, k]
    uint8_t *aq;                                // [T*k + T][2][ap] activation digits (pairs, then the shared expert's rows)
    float2 *asc;                                // [T*k + T][imax / 32] per chunk: scale, sum of the chunk's represented values
    uint32_t *ids_out;
    float *weights_out;
    uint32_t *sync;                             // counters (S_*), then the phase clocks of the first streaming CTA
    uint32_t *status;
    uint32_t partial_slices;                    // capacity of the partial-sum buffer (slices per CTA)
    uint32_t chain_ctas;                        // NC
    long long t0;                               // (device side) this CTA's clock at its start
    HcAdd hc;                                   // hyper-connection add applied where y is written (residual nullptr: none)
    uint32_t *status_mirror;                    // pinned host words [4] that receive the status words at the end, or nullptr
};

// One distinct source of phase C / one expert of phase B.
struct Src {
    uint16_t expert; uint8_t mask, shared;
    uint32_t slots;                             // slot of token t in byte t
    __device__ __forceinline__ uint32_t slot(uint32_t t) const { return (slots >> (8 * t)) & 0xffu; }
};

// Shared-memory plan of a streaming CTA (byte offsets), the same on host and device.  `region` is
// reused by the three phases; the digit image of x lives at its start through phases A and B.
struct FPlan {
    uint32_t bars, ids, wts, idx, wtx, misc, tokmask, slotmap, src, region, total;
    uint32_t kp;                                // pitch of one digit row of x
    uint32_t xq, xsum;                          // phases A and B (inside region)
    uint32_t xf, xf_pitch, rows, row_pitch;     // phase A
    uint32_t zs, ring, partial;                 // phase B
    uint32_t aq, ap, asc, tiles, cpartial;      // phase C
};
__host__ __device__ inline FPlan make_fplan(uint32_t hidden, uint32_t inter_max, uint32_t rows_c, uint32_t partial_slices) {
    FPlan p;
    uint32_t at = 0;
    p.bars = at; at += 512;
    p.ids = at; at += FTOK * FMAXK * 4;
    p.wts = at; at += FTOK * FMAXK * 4;
    p.idx = at; at += FTOK * FMAXK * 4;         // the exact routes as published
    p.wtx = at; at += FTOK * FMAXK * 4;
    p.misc = at; at += 1024;                    // floats [0..3] x maxima then scales, [4..7] shared logits; words from +64; +512: digitiser constants of x
    p.tokmask = at; at += FMAXE;
    p.slotmap = at; at += FMAXE * 4;
    p.src = at; at += ((FMAXSRC * 8 + 127) & ~127u);
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
    p.rows = a; a += FRMAX * p.row_pitch + 8 * 16 * 4;      // + the partial sums of the fast logits
    // phase B: the logit keys are dead before the first copy lands in the ring
    uint32_t b = head;
    p.zs = b;
    p.ring = b; b += FW * FNS * FSTAGE;
    if (b < head + FTOK * FZP * 4) b = head + FTOK * FZP * 4;
    p.partial = b; b += partial_slices * 256;
    // phase C
    uint32_t c = 0;
    p.ap = inter_max + 32;
    p.aq = c; c += rows_c * 2 * p.ap;
    c = (c + 127) & ~127u;
    p.asc = c; c += rows_c * (inter_max / 32) * 8;
    c = (c + 127) & ~127u;
    p.tiles = c; c += FW * FNC * FSTAGE;
    p.cpartial = c; c += FW * 32 * 8;
    uint32_t m = a > b ? a : b;
    m = m > c ? m : c;
    p.total = p.region + m;
    return p;
}
// Shared-memory plan of a chain CTA.
struct CPlan { uint32_t bars, misc, ids, wts, xf, xf_pitch, ring, zs, total; };
__host__ __device__ inline CPlan make_cplan(uint32_t hidden) {
    CPlan p;
    uint32_t at = 0;
    p.bars = at; at += 512;
    p.misc = at; at += 1024;
    p.ids = at; at += FMAXK * 4 * FTOK;
    p.wts = at; at += FMAXK * 4 * FTOK;
    p.xf_pitch = hidden * 4 + 16;
    p.xf = at; at += FTOK * p.xf_pitch;
    at = (at + 127) & ~127u;
    p.ring = at; at += CSTG * CROWS * CCH * 4;
    p.zs = at; at += FTOK * FZP * 4;
    p.total = at;
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
__device__ __forceinline__ void fbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fs_u32(bar)) : "memory");
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
// Rows [y, y + 8) of expert z, 32-bit words [x, x + box) of each, through a 3-D tensor map {words per row, rows per
// expert, experts}: one request for the eight row pieces of a unit slice, which lie a row apart in memory.
__device__ __forceinline__ void ftma_rows(void *dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(fs_u32(dst_smem)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(fs_u32(bar)) : "memory");
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
__device__ __forceinline__ void fred_release(uint32_t *p) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ void fmma_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Shared-memory loads by 32-bit shared address, volatile: they read memory that bulk copies rewrite between uses
// and must stay behind the mbarrier wait that precedes them in program order.
__device__ __forceinline__ uint2 lds_ring2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_ring_u16(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// Thread 0 waits until *counter >= expected (bounded); the verdict reaches every thread.
// False (CTA-uniform) when the wait ran out.
__device__ __forceinline__ bool wait_counter(const uint32_t *counter, uint32_t expected, uint32_t *status, uint32_t *flag_smem) {
    if (threadIdx.x == 0) {
        uint32_t ok = 1;
        const long long start = clock64();
        while (fld_acquire(counter) < expected) {
            if (clock64() - start > (1ll << 31)) { atomicOr(status, QW4SH_ERR_STATE); ok = 0; break; }
        }
        *flag_smem = ok;
    }
    __syncthreads();
    const bool ok = *flag_smem != 0;
    __syncthreads();
    return ok;
}
// All threads' earlier global writes are ordered before one release increment.
__device__ __forceinline__ void arrive_counter(uint32_t *counter) {
    __syncthreads();
    if (threadIdx.x == 0) fred_release(counter);
}

// ---- half blocks (128 columns) on the tensor cores ----------------------------------------------
// MMA k-slots are permuted so that lane (g, t) owns the eight consecutive columns 8t..8t+7 of
// every 32-column chunk, for MMA rows g and g + 8 and for activation column g (token g >> 1,
// digit g & 1).  f0 += row g . x[token t], f1 += row g+8 . x[token t].
//
// Halves (phase B): the activation has one scale per row, so the sums stay integers over a half
// block and the results are in units of the token's digit scale; xsum holds the token's digit
// sums (Q4_K's min term).
// HalvesS (phase C): one scale per 32-column chunk; `asc` points at the token row's (scale, chunk
// sum) pairs and the results are plain values.
template <uint32_t TYPE> struct Halves;
template <uint32_t TYPE> struct HalvesS;

__device__ __forceinline__ void q4k_scales(const uint4 h0, uint32_t hb, uint32_t &sc, uint32_t &mn) {
    if (hb == 0) { sc = h0.y & 0x3f3f3f3fu; mn = h0.z & 0x3f3f3f3fu; }
    else { sc = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u); mn = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u); }
}

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
            q4k_scales(h0, hb, sc0, mn0);
            q4k_scales(h1, hb, sc1, mn1);
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
template <> struct HalvesS<T_Q4_K> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, uint32_t halves, uint32_t, const uint16_t *,
                                            const uint16_t *, const uint8_t *, uint32_t t, const uint8_t *aq, const float2 *asc,
                                            float &f0, float &f1) {
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++, aq += 128, asc += 4) {
            const uint8_t *b0 = r0 + (h >> 1) * 144u, *b1 = r1 + (h >> 1) * 144u;
            const uint32_t hb = h & 1u;
            const uint4 h0 = *reinterpret_cast<const uint4 *>(b0), h1 = *reinterpret_cast<const uint4 *>(b1);
            uint32_t sc0, mn0, sc1, mn1;
            q4k_scales(h0, hb, sc0, mn0);
            q4k_scales(h1, hb, sc1, mn1);
            float qf0 = 0.0f, qf1 = 0.0f, mf0 = 0.0f, mf1 = 0.0f;
            const float lo = 1.0f / 254.0f;
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const uint2 q0 = *reinterpret_cast<const uint2 *>(b0 + 16 + (hb * 2 + cc) * 32 + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(b1 + 16 + (hb * 2 + cc) * 32 + 8 * t);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int j = cc * 2 + nib;
                    const uint2 bq = *reinterpret_cast<const uint2 *>(aq + j * 32);
                    int c[4];
                    fmma_zero(c, (q0.x >> (4 * nib)) & 0x0f0f0f0fu, (q1.x >> (4 * nib)) & 0x0f0f0f0fu,
                              (q0.y >> (4 * nib)) & 0x0f0f0f0fu, (q1.y >> (4 * nib)) & 0x0f0f0f0fu, bq.x, bq.y);
                    const float2 a = asc[j];
                    const float s0 = (float)((sc0 >> (8 * j)) & 0xffu), s1 = (float)((sc1 >> (8 * j)) & 0xffu);
                    const float m0 = (float)((mn0 >> (8 * j)) & 0xffu), m1 = (float)((mn1 >> (8 * j)) & 0xffu);
                    qf0 = fmaf(s0 * a.x, fmaf((float)c[1], lo, (float)c[0]), qf0);
                    qf1 = fmaf(s1 * a.x, fmaf((float)c[3], lo, (float)c[2]), qf1);
                    mf0 = fmaf(m0, a.y, mf0); mf1 = fmaf(m1, a.y, mf1);
                }
            }
            const float d0 = __half2float(__ushort_as_half((uint16_t)(h0.x & 0xffffu))), n0 = __half2float(__ushort_as_half((uint16_t)(h0.x >> 16)));
            const float d1 = __half2float(__ushort_as_half((uint16_t)(h1.x & 0xffffu))), n1 = __half2float(__ushort_as_half((uint16_t)(h1.x >> 16)));
            f0 += d0 * qf0 - n0 * mf0;
            f1 += d1 * qf1 - n1 * mf1;
        }
    }
};

// IQ2_XXS on this path is read from a second resident image, made at create (iq2_expand_kernel below): every
// weight as a 4-bit code (level | sign << 2), laid out for this kernel.  2.06 bits per weight become 4.5, and in
// exchange a lane turns eight weights into MMA operands with one shift and two byte permutes against an 8-byte
// table held in two registers (the codebook and sign look-ups of the packed form cost four shared-memory reads per
// eight weights and bound the whole kernel).  Decoded values are the same bits.
//
// Block of 512 columns, 288 bytes (the geometry of two Q4_K blocks, so slices, stages and tensor-map boxes are
// shared with that format):
//   [0, 256)    codes: the 32-bit word of lane t for 32-column chunk j of half h (columns 128 h + 32 j + 8 t .. + 7,
//               nibble i = column + i) sits at 64 h + 16 t + 4 j, so a lane reads its four chunks of a half with
//               one 128-bit load;
//   [256, 272)  2 * scale + 1 of the sixteen 32-column chunks, one byte each;
//   [272, 276)  the fp16 super-scales of the two 256-column source blocks;  [276, 288) zero.
constexpr uint32_t T_IQ2N = 116;                        // not a GGUF type: the expanded image of an IQ2_XXS tensor
constexpr uint32_t IQ2N_LO = 8u | 25u << 8 | 43u << 16 | 60u << 24;                                  // iq2_magnitude(0..3)
constexpr uint32_t IQ2N_HI = (256u - 8u) | (256u - 25u) << 8 | (256u - 43u) << 16 | (256u - 60u) << 24;   // the same, negated

__device__ __forceinline__ uint4 lds_ring4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_ring1(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

template <> struct Halves<T_IQ2N> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, uint32_t halves, uint32_t, const uint16_t *,
                                            const uint16_t *, const uint8_t *, uint32_t t, const uint8_t *xq, const int2 *,
                                            float &f0, float &f1) {
        const uint32_t a0s = fs_u32(r0) + 16u * t, a1s = fs_u32(r1) + 16u * t;
        uint32_t xs = fs_u32(xq);
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++, xs += 128) {
            const uint32_t at = (h >> 2) * 288u, hh = h & 3u;
            const uint4 w0 = lds_ring4(a0s + at + 64u * hh), w1 = lds_ring4(a1s + at + 64u * hh);
            const uint32_t s0 = lds_ring1(a0s - 16u * t + at + 256u + 4u * hh), s1 = lds_ring1(a1s - 16u * t + at + 256u + 4u * hh);
            const uint32_t dh0 = lds_ring_u16(a0s - 16u * t + at + 272u + (hh >> 1) * 2u), dh1 = lds_ring_u16(a1s - 16u * t + at + 272u + (hh >> 1) * 2u);
            const uint32_t c0[4] = {w0.x, w0.y, w0.z, w0.w}, c1[4] = {w1.x, w1.y, w1.z, w1.w};
            int iacc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 bq = lds_ring2(xs + j * 32);
                int c[4];
                fmma_zero(c, __byte_perm(IQ2N_LO, IQ2N_HI, c0[j]), __byte_perm(IQ2N_LO, IQ2N_HI, c1[j]),
                          __byte_perm(IQ2N_LO, IQ2N_HI, c0[j] >> 16), __byte_perm(IQ2N_LO, IQ2N_HI, c1[j] >> 16), bq.x, bq.y);
                const int k0 = (int)((s0 >> (8 * j)) & 0xffu), k1 = (int)((s1 >> (8 * j)) & 0xffu);               // 2 * scale + 1
                iacc[0] += c[0] * k0; iacc[1] += c[1] * k0; iacc[2] += c[2] * k1; iacc[3] += c[3] * k1;
            }
            const float lo = 1.0f / 254.0f;
            const float d0 = __half2float(__ushort_as_half((uint16_t)dh0)) * 0.125f, d1 = __half2float(__ushort_as_half((uint16_t)dh1)) * 0.125f;
            f0 += d0 * fmaf((float)iacc[1], lo, (float)iacc[0]);
            f1 += d1 * fmaf((float)iacc[3], lo, (float)iacc[2]);
        }
    }
};
template <> struct HalvesS<T_IQ2N> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, uint32_t halves, uint32_t, const uint16_t *,
                                            const uint16_t *, const uint8_t *, uint32_t t, const uint8_t *aq, const float2 *asc,
                                            float &f0, float &f1) {
        const uint32_t a0s = fs_u32(r0) + 16u * t, a1s = fs_u32(r1) + 16u * t;
        uint32_t xs = fs_u32(aq), ss = fs_u32(asc);
#pragma unroll 1
        for (uint32_t h = 0; h < halves; h++, xs += 128, ss += 32) {
            const uint32_t at = (h >> 2) * 288u, hh = h & 3u;
            const uint4 w0 = lds_ring4(a0s + at + 64u * hh), w1 = lds_ring4(a1s + at + 64u * hh);
            const uint32_t s0 = lds_ring1(a0s - 16u * t + at + 256u + 4u * hh), s1 = lds_ring1(a1s - 16u * t + at + 256u + 4u * hh);
            const uint32_t dh0 = lds_ring_u16(a0s - 16u * t + at + 272u + (hh >> 1) * 2u), dh1 = lds_ring_u16(a1s - 16u * t + at + 272u + (hh >> 1) * 2u);
            const uint32_t c0[4] = {w0.x, w0.y, w0.z, w0.w}, c1[4] = {w1.x, w1.y, w1.z, w1.w};
            float fa0 = 0.0f, fa1 = 0.0f;
            const float lo = 1.0f / 254.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 bq = lds_ring2(xs + j * 32), sc = lds_ring2(ss + j * 8);
                int c[4];
                fmma_zero(c, __byte_perm(IQ2N_LO, IQ2N_HI, c0[j]), __byte_perm(IQ2N_LO, IQ2N_HI, c1[j]),
                          __byte_perm(IQ2N_LO, IQ2N_HI, c0[j] >> 16), __byte_perm(IQ2N_LO, IQ2N_HI, c1[j] >> 16), bq.x, bq.y);
                const float k0 = (float)((s0 >> (8 * j)) & 0xffu), k1 = (float)((s1 >> (8 * j)) & 0xffu);       // 2 * scale + 1
                const float a = __uint_as_float(sc.x);
                fa0 = fmaf(k0 * a, fmaf((float)c[1], lo, (float)c[0]), fa0);
                fa1 = fmaf(k1 * a, fmaf((float)c[3], lo, (float)c[2]), fa1);
            }
            const float d0 = __half2float(__ushort_as_half((uint16_t)dh0)) * 0.125f, d1 = __half2float(__ushort_as_half((uint16_t)dh1)) * 0.125f;
            f0 = fmaf(d0, fa0, f0);
            f1 = fmaf(d1, fa1, f1);
        }
    }
};

// One thread per 32-column chunk of a row: the chunk's 32 codes, its scale byte, and (first chunk of a 256-column
// source block) the block's super-scale, from the resident IQ2_XXS image into the expanded one.
// which < 0: rows in order, [expert][row][blocks] (down tiles: sixteen rows are one contiguous span).  which = 0 / 1
// (gate / up): unit slices, [expert][unit of 8 rows][block][gate rows | up rows][288 bytes], so that the sixteen row
// pieces of one ring stage are ONE contiguous span of 4608 bytes.
__global__ void __launch_bounds__(256) iq2_expand_kernel(DevTensor t, uint8_t *__restrict__ out, int which) {
    const uint32_t nb = t.k_storage >> 8, chunks = t.k_storage >> 5;
    const uint64_t rows = (uint64_t)t.n_out * t.n_experts, total = rows * chunks;
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const uint64_t grow = i / chunks;                                          // expert * n_out + row
    const uint32_t q = (uint32_t)(i % chunks), expert = (uint32_t)(grow / t.n_out), row = (uint32_t)(grow % t.n_out);
    const uint8_t *mat = t.data + (uint64_t)expert * t.expert_bytes;
    const uint32_t blk = q >> 3, ch = q & 7u;
    const uint8_t *group = mat + ((uint64_t)row * nb * 8u + ((blk * 8u + ch) ^ iq2_swizzle(row, nb))) * 8u;
    const uint32_t bits = load_u32(group + 4);
    const uint32_t nb5 = t.k_storage >> 9;                                      // 512-column blocks per row
    uint8_t *block = which < 0 ? out + (grow * nb5 + (q >> 4)) * 288u           // the 512-column block of this chunk
                               : out + ((((uint64_t)expert * (t.n_out >> 3) + (row >> 3)) * nb5 + (q >> 4)) * 2u + (uint32_t)which) * 2304u + (row & 7u) * 288u;
    const uint32_t h = (q >> 2) & 3u, j = q & 3u;
    for (uint32_t slot = 0; slot < 4; slot++) {                                 // slot = lane t of the consumer: columns 8 t .. 8 t + 7
        const uint32_t levels = c_iq2_levels[group[slot]], signs = iq2_signs8((bits >> (7 * slot)) & 127u);
        uint32_t word = 0;
        for (uint32_t c = 0; c < 8; c++) word |= (((levels >> (2 * c)) & 3u) | (((signs >> c) & 1u) << 2)) << (4 * c);
        *reinterpret_cast<uint32_t *>(block + 64u * h + 16u * slot + 4u * j) = word;
    }
    block[256u + 4u * h + j] = (uint8_t)(2u * (bits >> 28) + 1u);
    if (ch == 0) {
        const uint64_t blocks = (uint64_t)t.n_out * nb;
        *reinterpret_cast<uint16_t *>(block + 272u + (blk & 1u) * 2u) = (uint16_t)load_u16(mat + blocks * 64u + ((uint64_t)row * nb + blk) * 2u);
    }
}

// Probe: rows [row0, row0 + rows) of one expert decoded FROM THE EXPANDED IMAGE into floats [rows, k], with the
// arithmetic of the reference's decoder (src/qwen4_packed.c:102-120: d * (2 s + 1) * 0.125 * magnitude, signed), so
// that the image can be compared bit for bit with a CPU decode of the GGUF bytes.  which as above.
__global__ void __launch_bounds__(256) iq2n_decode_rows_kernel(const uint8_t *__restrict__ image, uint32_t k, uint32_t n_out, uint32_t expert,
                                                               uint32_t row0, uint32_t rows, int which, float *__restrict__ out) {
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (uint64_t)rows * k) return;
    const uint32_t row = row0 + (uint32_t)(i / k), col = (uint32_t)(i % k), nb5 = k >> 9;
    const uint8_t *block = which < 0 ? image + (((uint64_t)expert * n_out + row) * nb5 + (col >> 9)) * 288u
                                     : image + ((((uint64_t)expert * (n_out >> 3) + (row >> 3)) * nb5 + (col >> 9)) * 2u + (uint32_t)which) * 2304u + (row & 7u) * 288u;
    const uint32_t c = col & 511u, h = c >> 7, j = (c >> 5) & 3u, t = (c >> 3) & 3u, n = c & 7u;
    const uint32_t word = *reinterpret_cast<const uint32_t *>(block + 64u * h + 16u * t + 4u * j), code = (word >> (4 * n)) & 15u;
    const uint32_t twice_plus_one = block[256u + 4u * h + j];
    const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(block + 272u + (h >> 1) * 2u));
    const float scale = __fmul_rn(__fmul_rn(d, (float)twice_plus_one), 0.125f);
    const float value = __fmul_rn(scale, (float)iq2_magnitude(code & 3u));
    out[i] = (code & 4u) ? -value : value;
}

// Geometry of one format inside the rings.
template <uint32_t TYPE> struct FGeo;
template <> struct FGeo<T_Q4_K> { static constexpr uint32_t SLICE_BLOCKS = 2, BLOCK_BYTES = 144; };      // 512 columns, 288 B per row
template <> struct FGeo<T_IQ2N> { static constexpr uint32_t SLICE_BLOCKS = 2, BLOCK_BYTES = 144; };      // the same: one 288-byte block of 512 columns

// Copies of slice `s` of a gate/up unit (8 gate rows + 8 up rows from row `row0` of expert `expert`) into `stage`:
// row r at r * slice bytes.  The eight row pieces of a
// matrix are ONE tensor-map request (issuing a request costs the warp about a hundred cycles whatever its size).
template <uint32_t TYPE>
__device__ __forceinline__ void issue_unit_slice(const CUtensorMap *gate_map, const CUtensorMap *up_map, const uint8_t *gate_mat,
                                              const uint8_t *up_mat, uint32_t expert, uint32_t n_out, uint32_t nb, uint32_t row0, uint32_t s,
                                              uint8_t *stage, uint64_t *bar, uint32_t lane) {
    constexpr uint32_t slice_bytes = FGeo<TYPE>::SLICE_BLOCKS * FGeo<TYPE>::BLOCK_BYTES;
    if (TYPE == T_IQ2N) {
        // the expanded image keeps a unit slice (gate rows, then up rows) as one span: gate_mat is the image's base
        if (lane == 0) {
            fbar_expect(bar, 16 * slice_bytes);
            fbulk(stage, gate_mat + ((((uint64_t)expert * (n_out >> 3) + (row0 >> 3)) * (nb >> 1) + s) * 16u) * slice_bytes, 16 * slice_bytes, bar);
        }
        return;
    }
    if (lane == 0) fbar_expect(bar, 16 * slice_bytes);
    __syncwarp();
    if (lane < 2) ftma_rows(stage + lane * 8 * slice_bytes, lane ? up_map : gate_map, s * (slice_bytes / 4), row0, expert, bar);
}
template <uint32_t TYPE>
__device__ __forceinline__ void consume_unit_slice(const uint8_t *stage, uint32_t nb, uint32_t s, const uint8_t *xq_lane,
                                                   const int2 *xsum_tok, uint32_t g, uint32_t t, float &f0, float &f1) {
    constexpr uint32_t SB = FGeo<TYPE>::SLICE_BLOCKS, slice_bytes = SB * FGeo<TYPE>::BLOCK_BYTES;
    const uint16_t *d = reinterpret_cast<const uint16_t *>(stage + 16 * slice_bytes);
    Halves<TYPE>::run(stage + g * slice_bytes, stage + (8 + g) * slice_bytes, SB * 2, iq2_swizzle(g, nb), d + g * nb + s * SB,
                      d + (8 + g) * nb + s * SB, nullptr, t, xq_lane + s * SB * 256u, xsum_tok + s * SB * 8u, f0, f1);
}

// Down tile: 16 rows x K (K <= 512), fetched whole.
template <uint32_t TYPE>
__device__ __forceinline__ void issue_down_tile(const uint8_t *mat, uint32_t n_out, uint32_t nb, uint32_t row0, uint8_t *stage, uint64_t *bar,
                                             uint32_t lane) {
    const uint32_t row_bytes = nb * FGeo<TYPE>::BLOCK_BYTES;
    if (lane == 0) {
        fbar_expect(bar, 16 * row_bytes);
        fbulk(stage, mat + row0 * row_bytes, 16 * row_bytes, bar);
    }
}
template <uint32_t TYPE>
__device__ __forceinline__ void consume_down_tile(const uint8_t *stage, uint32_t nb, const uint8_t *aq_lane,
                                                  const float2 *asc_tok, uint32_t g, uint32_t t, float &f0, float &f1) {
    const uint32_t row_bytes = nb * FGeo<TYPE>::BLOCK_BYTES;
    const uint16_t *d = reinterpret_cast<const uint16_t *>(stage + 4096);
    HalvesS<TYPE>::run(stage + g * row_bytes, stage + (8 + g) * row_bytes, nb * 2, iq2_swizzle(g, nb), d + g * nb, d + (8 + g) * nb, nullptr, t,
                       aq_lane, asc_tok, f0, f1);
}

// Two int8 digits per value: v ~ dx * (q1 + q2 / 254), |v| <= 127 dx.  Rounding by the
// 1.5 * 2^23 trick (no conversion instructions): the integer sits in the low mantissa bits, so
// the low byte of the rounded float's bit pattern IS the int8 digit.  c = (dx, 1 / dx, 254 / dx).
__device__ __forceinline__ void digit_pair(float v, const float4 c, uint32_t &ra, uint32_t &rb) {
    const float magic = 12582912.0f;
    const float r1 = fmaf(v, c.y, magic);
    const float q1 = r1 - magic;
    // second digit clamped to [-127, 127] in the float domain, before the rounding add
    const float r2 = fmaxf(-127.0f, fminf(127.0f, fmaf(-q1, c.x, v) * c.z)) + magic;
    ra = __float_as_uint(r1); rb = __float_as_uint(r2);
}
// Four values at once, packed; `s` accumulates both digit sums: the first in its low half, the
// second in its high half (each below 2^15 in magnitude for a 32-column chunk).
__device__ __forceinline__ void digits4(const float4 v, const float4 c, uint32_t &hi, uint32_t &lo, int &s) {
    const float vv[4] = {v.x, v.y, v.z, v.w};
    uint32_t ra[4], rb[4];
#pragma unroll
    for (int j = 0; j < 4; j++) digit_pair(vv[j], c, ra[j], rb[j]);
    hi = __byte_perm(__byte_perm(ra[0], ra[1], 0x0040), __byte_perm(ra[2], ra[3], 0x0040), 0x5410);
    lo = __byte_perm(__byte_perm(rb[0], rb[1], 0x0040), __byte_perm(rb[2], rb[3], 0x0040), 0x5410);
    s += __dp4a((int)hi, 0x01010101, 0) + (__dp4a((int)lo, 0x01010101, 0) << 16);
}

// Rows of `k` floats (k % 256 == 0) in shared memory with known maxima -> digit images, digit
// sums per 32-column chunk and scales.  A warp takes one 256-column segment of one row at a time:
// two float4 per lane, eight consecutive lanes cover one chunk.  `amax` holds the maxima on entry
// and the scales (max / 127, or 0 for an unusable row) on return; `consts` is scratch, one float4
// per row.  CTA-wide.
__device__ __forceinline__ void digitise_rows(const float *src, uint32_t src_pitch, uint32_t rows, uint32_t k, float *amax, uint8_t *dq,
                                           uint32_t dq_pitch, int2 *sums, uint32_t sums_pitch, float4 *consts) {
#pragma unroll 1
    for (uint32_t r = threadIdx.x; r < rows; r += FT) {
        const float m = amax[r];
        const bool usable = finite_f32(m) && m > 0.0f;
        const float inv = usable ? __fdividef(127.0f, m) : 0.0f;
        consts[r] = make_float4(usable ? m * (1.0f / 127.0f) : 0.0f, inv, 2.0f * inv * 127.0f, 0.0f);
    }
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, segs = k >> 8, units = rows * segs;
#pragma unroll 1
    for (uint32_t u = warp; u < units; u += FW) {
        const uint32_t r = u / segs, seg = u - r * segs;
        const float4 *from = reinterpret_cast<const float4 *>(src + (uint64_t)r * src_pitch) + seg * 64u + lane;
        const float4 v0 = *from, v1 = *(from + 32);
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
    __syncthreads();
#pragma unroll 1
    for (uint32_t r = threadIdx.x; r < rows; r += FT) amax[r] = consts[r].x;
    __syncthreads();
}

__device__ __forceinline__ float fast_sigmoid(float v) {
    const float e = __expf(-fabsf(v));
    return v >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
}

// Top-k of up to 32 * PL ordered keys held in registers, one warp: lane L holds the keys of elements
// L, L + 32, ... (0: absent).  Sequential selection (k dependent warp reductions) costs a lone warp
// several hundred cycles per round, so the work is arranged in parallel steps instead:
//   1. every lane's maximum, and the k-th largest of those 32 maxima: at least k elements reach it;
//   2. the elements that reach it (typically a dozen or two) are compacted into `cand` (shared memory);
//   3. every candidate counts the candidates that beat it (larger key, or equal key and lower element):
//      that count is its place, and places below k are written out.
// Returns false when more than 64 elements qualify (heavy ties): the caller then selects sequentially.
// cand: 128 words.  ids_out[place] = element, keys_out[place] = key (either may alias nothing else).
template <int PL>
__device__ __forceinline__ bool warp_topk(const uint32_t (&key)[PL], uint32_t lane, uint32_t k, uint32_t *cand, uint32_t *ids_out,
                                          uint32_t *keys_out) {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < PL; i++) m = max(m, key[i]);
    uint32_t ahead = 0;                                                     // lanes whose maximum beats this lane's
#pragma unroll
    for (int j = 0; j < 32; j++) {
        const uint32_t v = __shfl_sync(0xffffffffu, m, j);
        ahead += (v > m || (v == m && (uint32_t)j < lane)) ? 1u : 0u;
    }
    const uint32_t holder = __ballot_sync(0xffffffffu, ahead == min(k, 32u) - 1u);
    const uint32_t bound = max(__shfl_sync(0xffffffffu, m, __ffs(holder) - 1), 1u);
    uint32_t count = 0;
    const uint32_t below = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < PL; i++) {
        const bool in = key[i] >= bound;
        const uint32_t votes = __ballot_sync(0xffffffffu, in);
        const uint32_t at = count + __popc(votes & below);
        if (in && at < 64) { cand[at] = key[i]; cand[64 + at] = lane + 32u * i; }
        count += __popc(votes);
    }
    if (count > 64) return false;
    __syncwarp();
    const uint32_t k0 = lane < count ? cand[lane] : 0u, e0 = cand[64 + lane];
    const uint32_t k1 = lane + 32 < count ? cand[lane + 32] : 0u, e1 = cand[96 + lane];
    uint32_t place0 = 0, place1 = 0;
#pragma unroll 4
    for (uint32_t j = 0; j < count; j++) {
        const uint32_t kj = cand[j], ej = cand[64 + j];
        place0 += (kj > k0 || (kj == k0 && ej < e0)) ? 1u : 0u;
        place1 += (kj > k1 || (kj == k1 && ej < e1)) ? 1u : 0u;
    }
    if (lane < count && place0 < k) { ids_out[place0] = e0; if (keys_out) keys_out[place0] = k0; }
    if (lane + 32 < count && place1 < k) { ids_out[place1] = e1; if (keys_out) keys_out[place1] = k1; }
    __syncwarp();
    return true;
}
// The sequential form: every lane keeps its best three (key, element) pairs, so a selection step is one
// warp maximum and a ballot, and a lane rescans its registers only when it has won three times.
template <int PL>
__device__ __forceinline__ void topk_scan(const uint32_t (&key)[PL], uint32_t lane, uint32_t &b1, uint32_t &e1, uint32_t &b2, uint32_t &e2,
                                          uint32_t &b3, uint32_t &e3) {
    b1 = 0; e1 = 0xffffffffu; b2 = 0; e2 = 0xffffffffu; b3 = 0; e3 = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < PL; i++) {                                         // ascending element: the lowest wins among equals
        const uint32_t k = key[i], e = lane + 32u * i;
        if (k > b1) { b3 = b2; e3 = e2; b2 = b1; e2 = e1; b1 = k; e1 = e; }
        else if (k > b2) { b3 = b2; e3 = e2; b2 = k; e2 = e; }
        else if (k > b3) { b3 = k; e3 = e; }
    }
}
template <int PL>
__device__ __forceinline__ void topk_clear(uint32_t (&key)[PL], uint32_t index) {
#pragma unroll
    for (int i = 0; i < PL; i++) if ((uint32_t)i == index) key[i] = 0;
}
template <int PL>
__device__ __noinline__ void warp_topk_sequential(uint32_t (&key)[PL], uint32_t lane, uint32_t k, uint32_t *ids_out, uint32_t *keys_out) {
    uint32_t b1, e1, b2, e2, b3, e3, spare = 2;
    topk_scan<PL>(key, lane, b1, e1, b2, e2, b3, e3);
#pragma unroll 1
    for (uint32_t slot = 0; slot < k; slot++) {
        const uint32_t top = __reduce_max_sync(0xffffffffu, b1);
        const uint32_t e_win = __reduce_min_sync(0xffffffffu, b1 == top ? e1 : 0xffffffffu);
        if (lane == 0) { ids_out[slot] = e_win; if (keys_out) keys_out[slot] = top; }
        if ((e_win & 31u) == lane) {
            topk_clear<PL>(key, e_win >> 5);
            if (spare) { b1 = b2; e1 = e2; b2 = b3; e2 = e3; spare--; }
            else { topk_scan<PL>(key, lane, b1, e1, b2, e2, b3, e3); spare = 2; }
        }
    }
    __syncwarp();
}

// Softmax, top-k and renormalisation of ONE row of logits in shared memory (zs), CTA-wide;
// src/qwen4_moe.c:209-247 with its order of operations: ties go to the lower id, and with `exact`
// the exp-sum runs serially over e = 0..E-1 (the reference's bits); otherwise it is a warp tree
// sum.  Returns false (CTA-uniform) when a logit is not finite; the row is recorded.
__device__ __forceinline__ bool route_row(float *zs, uint32_t E, uint32_t k, int norm, uint32_t row, bool exact, uint32_t *ids_s, float *wts_s,
                                       float *scratch, const unsigned long long *exp_table, uint32_t *flag, uint32_t *status) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid == 0) *flag = 1;
    __syncthreads();
    if (warp == 0) {                                                      // row maximum and finiteness
        float m = -CUDART_INF_F;
        bool bad = false;
#pragma unroll 4
        for (uint32_t e = lane; e < E; e += 32) { const float v = zs[e]; bad |= !finite_f32(v); m = fmaxf(m, v); }
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        bad = __any_sync(0xffffffffu, bad);
        if (lane == 0) {
            scratch[0] = m;
            if (bad) { atomicOr(status, QW4SH_ERR_NONFINITE); atomicMin(status + 1, row); *flag = 0; }
        }
    }
    __syncthreads();
    if (!*flag) return false;
    {
        const float m = scratch[0];
#pragma unroll 1
        for (uint32_t e = tid; e < E; e += FT) zs[e] = expf_libm_table(__fsub_rn(zs[e], m), exp_table);   // p = expf(z - max)
    }
    __syncthreads();
    if (warp == 0) {
        float sum = 0.0f;
        if (exact) {
            if (lane == 0) {                                               // the reference's serial sum
                // 32 values per pass: the loads of the next pass are issued before the 32 dependent adds of this
                // one, and the loop overhead hides under the add chain
                uint32_t e = 0;
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = E >= 32 ? *reinterpret_cast<const float4 *>(zs + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (; e + 32 <= E; e += 32) {
                    float4 w[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) w[j] = e + 64 <= E ? *reinterpret_cast<const float4 *>(zs + e + 32 + 4 * j) : v[j];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        sum = __fadd_rn(sum, v[j].x); sum = __fadd_rn(sum, v[j].y); sum = __fadd_rn(sum, v[j].z); sum = __fadd_rn(sum, v[j].w);
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = w[j];
                }
                for (; e < E; e++) sum = __fadd_rn(sum, zs[e]);
            }
            sum = __shfl_sync(0xffffffffu, sum, 0);
        } else {
#pragma unroll 4
            for (uint32_t e = lane; e < E; e += 32) sum += zs[e];
            for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (lane == 0) scratch[1] = sum;
    }
    __syncthreads();
    {
        const float sum = scratch[1];
#pragma unroll 1
        for (uint32_t e = tid; e < E; e += FT) zs[e] = __fdiv_rn(zs[e], sum);
    }
    __syncthreads();
    if (warp == 0) {
        // keys: bits of p / sum (>= 0, so ordered as integers) + 1
        constexpr int PL = FMAXE / 32;
        uint32_t key[PL];
#pragma unroll
        for (int i = 0; i < PL; i++) { const uint32_t e = lane + 32u * i; key[i] = e < E ? __float_as_uint(zs[e]) + 1u : 0u; }
        __syncwarp();
        uint32_t *cand = reinterpret_cast<uint32_t *>(zs), *keys_out = cand + 128;     // the probabilities are in registers now
        if (!warp_topk<PL>(key, lane, k, cand, ids_s, keys_out)) warp_topk_sequential<PL>(key, lane, k, ids_s, keys_out);
        const float mine = lane < k ? __uint_as_float(keys_out[lane] - 1u) : 0.0f;
        float selected = 0.0f;
#pragma unroll 1
        for (uint32_t slot = 0; slot < k; slot++) selected = __fadd_rn(selected, __shfl_sync(0xffffffffu, mine, slot));   // slot order
        if (lane < k) wts_s[lane] = norm ? __fdiv_rn(mine, selected) : mine;
    }
    __syncthreads();
    return true;
}

// The k largest of one row of logits by VALUE (ties to the lower id), one warp; the row is turned
// read into ordered integer keys (its memory then serves as scratch).  `extra`: choose k + 1 and put the last one in slot k - 1 (a
// deliberately wrong set, for the test of the repair path).  Returns false on a nonfinite logit.
__device__ __forceinline__ bool speculate_row(float *zs, uint32_t E, uint32_t k, bool extra, uint32_t *ids_s, uint32_t lane) {
    constexpr int PL = FMAXE / 32;
    uint32_t key[PL];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < PL; i++) {
        const uint32_t e = lane + 32u * i;
        const uint32_t u = e < E ? __float_as_uint(zs[e]) : 0u;
        bad |= e < E && (u & 0x7f800000u) == 0x7f800000u;
        key[i] = e < E ? ((u & 0x80000000u) ? ~u : (u | 0x80000000u)) : 0u;      // monotone in the value, never 0
    }
    if (__any_sync(0xffffffffu, bad)) return false;
    __syncwarp();
    uint32_t *cand = reinterpret_cast<uint32_t *>(zs);                          // the row is in registers now
    const uint32_t want = extra && k < E ? k + 1 : k;
    uint32_t *out = extra ? cand + 128 : ids_s;
    if (!warp_topk<PL>(key, lane, want, cand, out, nullptr)) warp_topk_sequential<PL>(key, lane, want, out, nullptr);
    if (extra) {                                                                // the wrong set: the (k + 1)-th takes the k-th's place
        if (lane < k) ids_s[lane] = out[lane == k - 1 && want > k ? k : lane];
        __syncwarp();
    }
    return true;
}

// CLOCK: SM clock of the first streaming CTA at a phase boundary.  MARK: cycles since its own start, for every CTA
// (words S_MARKS + 4 * cta + i of the sync array).
#ifdef QW4_NO_PHASE_CLOCKS
#define CLOCK(i) do { } while (0)
#define MARK(i) do { } while (0)
#else
#define CLOCK(i) do { if (clocked) clocks[i] = clock64(); } while (0)
#define MARK(i) do { if (threadIdx.x == 0) a.sync[S_MARKS + 4 * blockIdx.x + (i)] = (uint32_t)(clock64() - a.t0); } while (0)
#endif

// ---- chain CTA -----------------------------------------------------------------------------------
// Exact logits of router rows [32 c, 32 c + 32) (row E is the shared expert's router) for every
// token, then, in CTA t < T, the routing of token t.
__device__ __forceinline__ void chain_cta(FusedArgs &a, uint8_t *smem) {
    const uint32_t T = a.tokens, H = a.hidden, E = a.experts, k = a.top_k;
    const CPlan p = make_cplan(H);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, cta = blockIdx.x;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + p.bars);              // [CSTG]
    uint64_t *empty = full + CSTG;                                             // [CSTG]
    uint64_t *xbar = empty + CSTG;
    float *misc_f = reinterpret_cast<float *>(smem + p.misc);
    uint32_t *misc_u = reinterpret_cast<uint32_t *>(smem + p.misc) + 16;
    unsigned long long *exp_table = reinterpret_cast<unsigned long long *>(smem + p.misc + 256);
    const bool exact = a.router_mode != 1;
    const uint32_t loaders = 64;                                               // two loader warps: the rest sleep at the CTA barrier
    if (tid < CSTG) { fbar_init(&full[tid], loaders); fbar_init(&empty[tid], T); }
    if (tid == CSTG) fbar_init(xbar, 1);
    if (tid <= CSTG) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (tid < 32) exp_table[tid] = c_exp2_table[tid];
    __syncthreads();
    const uint32_t r0 = cta * CROWS;
    const uint32_t nr = exact && r0 <= E ? min((uint32_t)CROWS, E + 1 - r0) : 0;
    bool alive = true;
    if (nr && warp >= T && warp < T + 2) {
        // loader warps (weights only: they start before the previous launch has drained): 16-byte pieces of the
        // chunk, piece q of row r stored at position q ^ (r & 7)
        uint8_t *ring = smem + p.ring;
        const uint32_t lt = tid - 32 * T, pieces = nr * (CCH / 4), chunks = H / CCH;
#pragma unroll 1
        for (uint32_t i = 0; i < chunks && alive; i++) {
            const uint32_t st = i % CSTG;
            if (i >= CSTG) {
                const uint32_t parity = ((i / CSTG) - 1u) & 1u;
                const long long start = clock64();
                while (!fbar_try(&empty[st], parity)) {                         // the chain warps share the schedulers: poll gently
                    __nanosleep(200);
                    if (clock64() - start > (1ll << 31)) { atomicOr(a.status, QW4SH_ERR_STATE); alive = false; break; }
                }
            }
            if (!alive) break;
#pragma unroll 1
            for (uint32_t pc = lt; pc < pieces; pc += loaders) {
                const uint32_t r = pc / (CCH / 4), q = pc % (CCH / 4), gr = r0 + r;
                const uint8_t *src = (gr < E ? a.w[0].data + (uint64_t)gr * a.w[0].row_bytes : a.w[7].data) + (uint64_t)i * (CCH * 4) + q * 16u;
                const uint32_t dst = fs_u32(ring + (st * CROWS + r) * (CCH * 4) + ((q ^ (r & 7u)) << 4));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(fs_u32(&full[st])) : "memory");
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) a.t0 = clock64();                                            // read back by thread 0 only
    if (nr && warp < T) {
        // chain warp: token = warp, lane = row.  Multiplies and adds are separately rounded.
        uint8_t *xf = smem + p.xf;
        const uint8_t *ring = smem + p.ring;
        const uint32_t chunks = H / CCH;
        if (tid == 0) {
            fbar_expect(xbar, T * H * 4u);
            for (uint32_t q = 0; q < T; q++) fbulk(xf + q * p.xf_pitch, a.x + (uint64_t)q * H, H * 4u, xbar);
        }
        alive = fbar_wait(xbar, 0, a.status);
        MARK(2);
        long long waited = 0;
        const float4 *xv = reinterpret_cast<const float4 *>(xf + warp * p.xf_pitch);
        float sum = 0.0f;
#pragma unroll 1
        for (uint32_t i = 0; i < chunks; i++) {
            const uint32_t st = i % CSTG;
            const long long w0 = clock64();
            if (alive) alive = fbar_wait(&full[st], (i / CSTG) & 1u, a.status);
            alive = __all_sync(0xffffffffu, alive);
            waited += clock64() - w0;
            if (!alive) break;
            const uint8_t *row = ring + (st * CROWS + lane) * (CCH * 4);
            // a lone warp issues every other cycle: the products go two at a time (mul.rn.f32x2 rounds each half
            // like a scalar multiply), which leaves load + 2 packed multiplies + 4 adds per four columns, just
            // under the adds' own latency
#pragma unroll
            for (uint32_t q = 0; q < CCH / 4; q++) {
                const ulonglong2 w4 = *reinterpret_cast<const ulonglong2 *>(row + ((q ^ (lane & 7u)) << 4));
                const ulonglong2 x4 = *reinterpret_cast<const ulonglong2 *>(&xv[i * (CCH / 4) + q]);
                unsigned long long p01, p23;
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p01) : "l"(w4.x), "l"(x4.x));
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p23) : "l"(w4.y), "l"(x4.y));
                sum = __fadd_rn(sum, __uint_as_float((uint32_t)p01)); sum = __fadd_rn(sum, __uint_as_float((uint32_t)(p01 >> 32)));
                sum = __fadd_rn(sum, __uint_as_float((uint32_t)p23)); sum = __fadd_rn(sum, __uint_as_float((uint32_t)(p23 >> 32)));
            }
            __syncwarp();
            if (lane == 0) fbar_arrive(&empty[st]);
        }
        if (alive && lane < nr) {
            const uint32_t r = r0 + lane;
            if (!finite_f32(sum)) { atomicOr(a.status, QW4SH_ERR_NONFINITE); atomicMin(a.status + 1, warp); }
            if (r < E) a.logits[(uint64_t)warp * E + r] = sum; else a.shared_logit[warp] = sum;
        }
        if (tid == 0) a.sync[S_MARKS + 4 * blockIdx.x + 3] = (uint32_t)waited;
    }
    MARK(0);
    if (exact) arrive_counter(a.sync + S_CHAIN);          // also for a CTA without rows: the count is NC
    if (cta >= T) return;
    // ---- routing of token `cta` ----
    const uint32_t waited = exact ? S_CHAIN : S_FAST;
    const uint32_t expected = exact ? a.chain_ctas : gridDim.x - a.chain_ctas;
    bool ok = wait_counter(a.sync + waited, expected, a.status, misc_u);
    float *zs = reinterpret_cast<float *>(smem + p.zs);
    uint32_t *ids_s = reinterpret_cast<uint32_t *>(smem + p.ids);
    float *wts_s = reinterpret_cast<float *>(smem + p.wts);
    if (ok) {
        const float *from = exact ? a.logits + (uint64_t)cta * E : a.logits_fast + (uint64_t)cta * a.fast_pitch;
#pragma unroll 1
        for (uint32_t e = tid; e < E; e += FT) {
            const float v = __ldcg(from + e);
            zs[e] = v;
            if (!exact) a.logits[(uint64_t)cta * E + e] = v;
        }
        if (!exact && tid == 0) a.shared_logit[cta] = __ldcg(a.logits_fast + (uint64_t)cta * a.fast_pitch + E);
        __syncthreads();
        ok = route_row(zs, E, k, a.norm, cta, exact, ids_s, wts_s, misc_f + 8, exp_table, misc_u + 1, a.status);
    }
    if (ok && tid < k) {
        const uint32_t e = ids_s[tid];
        const float w = wts_s[tid];
        a.ids[cta * k + tid] = e; a.weights[cta * k + tid] = w;
        if (a.ids_out) a.ids_out[cta * k + tid] = e;
        if (a.weights_out) a.weights_out[cta * k + tid] = w;
    }
    if (!ok && tid == 0) atomicOr(a.sync + S_ROUTE_FAIL, 1u);
    __threadfence();
    arrive_counter(a.sync + S_ROUTED);
    MARK(1);
}

// ---- the kernel ---------------------------------------------------------------------------------
template <uint32_t RT, uint32_t ST>
__global__ void __launch_bounds__(FT, 1) fused_decode_kernel(const __grid_constant__ FusedArgs args, const __grid_constant__ CUtensorMap map_g,
                                                             const __grid_constant__ CUtensorMap map_u, const __grid_constant__ CUtensorMap map_sg,
                                                             const __grid_constant__ CUtensorMap map_su) {
    extern __shared__ __align__(128) uint8_t smem[];
    // The arguments span several cache lines of the constant bank, and a first touch of each line
    // costs a miss that every SM takes at the same moment.  All lines are fetched at once here,
    // into shared memory, and read from there afterwards.
    __shared__ FusedArgs a;
    for (uint32_t i = threadIdx.x; i < sizeof(FusedArgs) / 4; i += FT)
        reinterpret_cast<uint32_t *>(&a)[i] = reinterpret_cast<const uint32_t *>(&args)[i];
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t NC = a.chain_ctas;
    const uint32_t tid = threadIdx.x;
    __shared__ uint32_t leaving_last;
    auto leave = [&]() {
        // the CTA that leaves last clears the counters for the next launch
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            leaving_last = atomicAdd(a.sync + S_EXITS, 1u) == gridDim.x - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (leaving_last && tid < 8) { a.sync[tid] = 0; __threadfence(); }
        // every CTA's error bits are in before its exit count: the last one hands the words to the host
        if (leaving_last && tid < 4 && a.status_mirror) a.status_mirror[tid] = *reinterpret_cast<volatile uint32_t *>(a.status + tid);
    };
    if (blockIdx.x < NC) { chain_cta(a, smem); leave(); return; }

    const uint32_t T = a.tokens, H = a.hidden, E = a.experts, k = a.top_k, I = a.inter, IS = a.shared_inter;
    const uint32_t pairs = T * k, rows_c = pairs + T, imax = I > IS ? I : IS;
    const FPlan p = make_fplan(H, imax, rows_c, a.partial_slices);
    const uint32_t warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t sc = blockIdx.x - NC, NS = gridDim.x - NC;
    uint64_t *ringbar = reinterpret_cast<uint64_t *>(smem + p.bars);           // [FW][FNS], four single ones, then [FW][FNC]
    uint64_t *rowbar = ringbar + FW * FNS;
    uint64_t *tilebar = ringbar + FW * FNS + 4 + (threadIdx.x >> 5) * FNC;     // this warp's barriers of the down phase
    static_assert((FW * FNS + 4 + FW * FNC) * 8 <= 512, "the barrier block is 512 bytes");
    uint64_t *lutbar = rowbar + 1;
    uint64_t *xbar = lutbar + 1;                                               // x rows (phase A), then the fast logits (phase B)
    uint64_t *abar = xbar + 1;                                                 // activation digits (phase C)
    uint32_t *ids_s = reinterpret_cast<uint32_t *>(smem + p.ids);              // the ids phase B works with
    float *wts_s = reinterpret_cast<float *>(smem + p.wts);                    // exact weights in the order of ids_s
    uint32_t *ids_x = reinterpret_cast<uint32_t *>(smem + p.idx);              // the exact routes as published
    float *wts_x = reinterpret_cast<float *>(smem + p.wtx);
    float *misc_f = reinterpret_cast<float *>(smem + p.misc);                  // [0..3] x maxima then scales, [4..7] shared logits
    uint32_t *misc_u = reinterpret_cast<uint32_t *>(smem + p.misc) + 16;       // [0] wait flag, [1] spec ok, [2] sources, [3] verify, [4..19] chunk counts
    uint8_t *tokmask = smem + p.tokmask, *slotmap = smem + p.slotmap;
    Src *srcs = reinterpret_cast<Src *>(smem + p.src);
    uint8_t *region = smem + p.region;
    uint8_t *xq = region + p.xq;
    int2 *xsum = reinterpret_cast<int2 *>(region + p.xsum);
    unsigned long long *clocks = reinterpret_cast<unsigned long long *>(a.sync + S_CLOCKS);
    const bool clocked = sc == 0 && tid == 0;

    if (tid < FW * FNS + 4 + FW * FNC) {                                       // the barriers lie one after the other: one thread each
        fbar_init(&ringbar[tid], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 8) misc_f[tid] = 0.0f;
    float4 *xconsts = reinterpret_cast<float4 *>(smem + p.misc + 512);
    __syncthreads();

    // ================================ phase A ================================
    const uint32_t n_rows = sc <= E ? (E - sc) / NS + 1 : 0;                  // router rows sc, sc + NS, ... <= E
    uint8_t *xf = region + p.xf;
    uint8_t *rows = region + p.rows;
    // weights first: nothing another launch writes
    if (warp == 0) {
        if (lane == 0) fbar_expect(rowbar, n_rows * H * 4u);
        __syncwarp();
        if (lane < n_rows) {
            const uint32_t r = sc + lane * NS;
            const uint8_t *src = r < E ? a.w[0].data + (uint64_t)r * a.w[0].row_bytes : a.w[7].data;
            fbulk(rows + lane * p.row_pitch, src, H * 4u, rowbar);
        }
    } else if (warp == 1 && lane < 3) {                                        // the shared expert's tensors -> L2: one request per tensor
        const uint32_t m = 4 + lane;
        const uint32_t bytes = (uint32_t)a.w[m].expert_bytes & ~15u;            // shared tensors are far below 4 GB
        const uint32_t sub = ((bytes / NS) + 16u) & ~15u;
        const uint32_t from = sc * sub;
        if (from < bytes) fprefetch_l2(a.w[m].data + from, from + sub <= bytes ? sub : bytes - from);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) a.t0 = clock64();
    CLOCK(0);
    if (warp == 0) {
        if (lane == 0) fbar_expect(xbar, T * H * 4u);
        __syncwarp();
        if (lane < T) fbulk(xf + lane * p.xf_pitch, a.x + (uint64_t)lane * H, H * 4u, xbar);
    }
    // x -> shared memory (float, one bulk copy per row) with the row maxima, then digits; token rows beyond T stay zero
    bool alive = fbar_wait(xbar, 0, a.status);
    CLOCK(1);
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
#pragma unroll 1
        for (uint32_t i = tid; i < (FTOK - T) * 2 * (p.kp >> 4); i += FT)       // digit rows of absent tokens
            reinterpret_cast<uint4 *>(xq + 2 * T * p.kp)[i] = make_uint4(0, 0, 0, 0);
#pragma unroll 1
        for (uint32_t i = tid; i < (FTOK - T) * (H >> 5); i += FT) xsum[T * (H >> 5) + i] = make_int2(0, 0);
    }
    __syncthreads();
    // tree-summed logits of this CTA's rows: eight warps split K, each holds its columns of x in registers
    // and reads every router row once; sixteen (row, token) sums per warp, then eight partial sums each
    if (alive) alive = fbar_wait(rowbar, 0, a.status);
    float *lpart = reinterpret_cast<float *>(region + p.rows + FRMAX * p.row_pitch);    // [8 warps][16]
    if (warp < 8 && alive) {
        float acc[FRMAX][FTOK];
#pragma unroll
        for (int j = 0; j < FRMAX; j++)
#pragma unroll
            for (int q = 0; q < FTOK; q++) acc[j][q] = 0.0f;
        const uint32_t per_warp = H >> 3;                                      // columns of this warp
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < per_warp; c0 += 128) {
            const uint32_t col = warp * per_warp + c0 + lane * 4;
            float4 xv[FTOK];
#pragma unroll
            for (int q = 0; q < FTOK; q++)
                xv[q] = (uint32_t)q < T ? *reinterpret_cast<const float4 *>(xf + q * p.xf_pitch + col * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < FRMAX; j++) {
                if ((uint32_t)j < n_rows) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(rows + j * p.row_pitch + col * 4);
#pragma unroll
                    for (int q = 0; q < FTOK; q++)
                        acc[j][q] = fmaf(w4.x, xv[q].x, fmaf(w4.y, xv[q].y, fmaf(w4.z, xv[q].z, fmaf(w4.w, xv[q].w, acc[j][q]))));
                }
            }
        }
#pragma unroll
        for (int j = 0; j < FRMAX; j++)
#pragma unroll
            for (int q = 0; q < FTOK; q++) {
                float v = acc[j][q];
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) lpart[warp * 16 + j * FTOK + q] = v;
            }
    }
    __syncthreads();
    if (tid < n_rows * FTOK && (tid % FTOK) < T && alive) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++) v += lpart[w * 16 + tid];
        a.logits_fast[(uint64_t)(tid % FTOK) * a.fast_pitch + sc + (tid / FTOK) * NS] = v;
    }
    CLOCK(2);
    arrive_counter(a.sync + S_FAST);                                          // (its CTA barrier also orders the reads of xf before the digits' consts)
    digitise_rows(reinterpret_cast<const float *>(xf), p.xf_pitch >> 2, T, H, misc_f, xq, p.kp, xsum, H >> 5, xconsts);
    CLOCK(3);
    if (!wait_counter(a.sync + S_FAST, NS, a.status, misc_u)) return;
    CLOCK(4);
    MARK(0);

    // ================================ phase B ================================
    float *zs = reinterpret_cast<float *>(region + p.zs);
    if (warp == 0 && alive) {
        asm volatile("fence.proxy.async;" ::: "memory");                          // generic-proxy writes (the logits; phase A's use of this memory) before the copy
        if (lane == 0) fbar_expect(xbar, T * a.fast_pitch * 4u);
        __syncwarp();
        if (lane < T) fbulk(zs + lane * FZP, a.logits_fast + (uint64_t)lane * a.fast_pitch, a.fast_pitch * 4u, xbar);
    }
    if (alive) alive = fbar_wait(xbar, 1, a.status);                           // second use of this barrier: phase parity 1
    CLOCK(13);
    if (tid == 0) misc_u[1] = 1;
    __syncthreads();
    if (warp < T) {
        if (a.router_mode == 1 && lane == 0) misc_f[4 + warp] = zs[warp * FZP + E];     // the shared router's tree sum
        CLOCK(14);
        const bool fine = speculate_row(zs + warp * FZP, E, k, a.router_mode == 2 && warp == 0, ids_s + warp * k, lane);
        if (!fine && lane == 0) misc_u[1] = 0;
        CLOCK(15);
    }
    __syncthreads();
    const bool all_alive = __syncthreads_and(alive);
    bool lists_ok = misc_u[1] != 0 && all_alive;
    CLOCK(5);

    uint32_t ring_count = 0;                                                   // slices this warp has pushed through its ring
    uint64_t *bar = ringbar + warp * FNS;
    uint32_t n_src = 0;
    const uint32_t gs = IS >> 5, gr = I >> 5;                                  // granules (32 activation columns) per expert
    const uint32_t nbh = H >> 8;
    const uint32_t spu_s = nbh / FGeo<ST>::SLICE_BLOCKS, spu_r = nbh / FGeo<RT>::SLICE_BLOCKS;
#pragma unroll 1
    for (uint32_t attempt = 0; attempt < 2; attempt++) {
        // ---- lists from ids_s: token masks and slots per expert, distinct experts in ascending order behind the shared expert ----
        if (lists_ok) {
            if (warp == 0) {                                                   // one warp, warp-level synchronisation only
#pragma unroll 1
                for (uint32_t i = lane; i < FMAXE / 4; i += 32) reinterpret_cast<uint32_t *>(tokmask)[i] = 0;
                __syncwarp();
#pragma unroll 1
                for (uint32_t pr = lane; pr < pairs; pr += 32) {
                    const uint32_t e = ids_s[pr], tok = pr / k;
                    atomicOr(reinterpret_cast<uint32_t *>(tokmask) + (e >> 2), (1u << tok) << (8 * (e & 3u)));
                    slotmap[e * 4 + tok] = (uint8_t)(pr % k);
                }
                __syncwarp();
                if (lane == 0) { Src s0; s0.expert = 0xffffu; s0.mask = (uint8_t)((1u << T) - 1u); s0.shared = 1; s0.slots = 0; srcs[0] = s0; }
                uint32_t running = 1;
#pragma unroll 4
                for (uint32_t c = 0; c < (E + 31) / 32; c++) {
                    const uint32_t e = c * 32 + lane;
                    const bool has = e < E && tokmask[e] != 0;
                    const uint32_t any = __ballot_sync(0xffffffffu, has);
                    if (has) {
                        Src sn; sn.expert = (uint16_t)e; sn.mask = tokmask[e]; sn.shared = 0;
                        sn.slots = *reinterpret_cast<const uint32_t *>(slotmap + e * 4);
                        srcs[running + __popc(any & ((1u << lane) - 1u))] = sn;
                    }
                    running += __popc(any);
                }
                if (lane == 0) misc_u[2] = running;
            }
            __syncthreads();
            n_src = misc_u[2];
        }
        CLOCK(6);
        if (lists_ok) {
            // ---- gate/up: whole granules per CTA, the shared expert's first ----
            const uint32_t total = gs + (n_src - 1) * gr;
            const uint32_t g0 = total * sc / NS, g1 = total * (sc + 1) / NS;               // total <= 65 * 32: no overflow
            const uint32_t n_shg = g0 < gs ? min(gs, g1) - g0 : 0;               // shared granules of this CTA come first
            const uint32_t n_shu = n_shg * 4;
            const uint32_t slices = min(n_shu * spu_s + ((g1 - g0) * 4 - n_shu) * spu_r, a.partial_slices);
            const uint32_t mine = slices > warp ? (slices - 1 - warp) / FW + 1 : 0;
            uint8_t *ring = region + p.ring + warp * FNS * FSTAGE;
            float2 *partial = reinterpret_cast<float2 *>(region + p.partial);
            alive = __all_sync(0xffffffffu, alive);
            // CTA slice n -> local unit, slice, kind.  Both formats cut a unit into the same number of slices; the
            // divisors are powers of two for every shape met so far, and a runtime division costs a lone lane as
            // much as a quarter of a slice's arithmetic.
            const uint32_t spu = spu_r, spu_sh = (spu & (spu - 1u)) ? 32u : 31u - (uint32_t)__clz(spu);
            const uint32_t ur = gr * 4, ur_sh = (ur & (ur - 1u)) ? 32u : 31u - (uint32_t)__clz(ur);
            auto locate = [&](uint32_t n, uint32_t &ul, uint32_t &s, bool &sh) {
                if (spu_sh < 32u) { ul = n >> spu_sh; s = n & (spu - 1u); } else { ul = n / spu; s = n - ul * spu; }
                sh = ul < n_shu;
            };
            auto issue = [&](uint32_t i) {
                uint32_t ul, s; bool sh;
                locate(warp + i * FW, ul, s, sh);
                const uint32_t u = g0 * 4 + ul;                                    // unit index over all sources
                const uint32_t at = ring_count + i;
                uint8_t *stage = ring + (at % FNS) * FSTAGE;
                if (sh) issue_unit_slice<ST>(&map_sg, &map_su, a.w[4].data, a.w[5].data, 0, IS, nbh, u * 8, s, stage, &bar[at % FNS], lane);
                else {
                    const uint32_t v = u - gs * 4, vq = ur_sh < 32u ? v >> ur_sh : v / ur, e = srcs[1 + vq].expert;
                    issue_unit_slice<RT>(&map_g, &map_u, a.w[1].data, a.w[2].data, e, I, nbh, (v - vq * ur) * 8, s, stage, &bar[at % FNS], lane);
                }
            };
            __syncthreads();                                                       // the keys in zs are dead: the ring may be written
            fproxy_fence();
            if (alive) for (uint32_t i = 0; i < FNS && i < mine; i++) issue(i);
            // down tiles of this CTA's columns -> L2, ahead of phase C
#pragma unroll 1
            for (uint32_t tile = sc; tile < (H >> 4); tile += NS)
                for (uint32_t j = warp * 4 + lane; lane < 4 && j < n_src; j += FW * 4) {      // a few requests per warp: none of them falls behind
                    const Src s = srcs[j];
                    const uint32_t rb = (s.shared ? IS >> 8 : I >> 8) * 144u;
                    const uint8_t *mat = s.shared ? a.w[6].data : a.w[3].data + (uint64_t)s.expert * a.w[3].expert_bytes;
                    fprefetch_l2(mat + tile * 16 * rb, 16 * rb);
                }
            const uint8_t *xq_lane = xq + g * p.kp + 8 * t;
            const int2 *xsum_tok = xsum + t * (H >> 5);
#pragma unroll 1
            for (uint32_t i = 0; i < mine; i++) {
                uint32_t ul, s; bool sh;
                locate(warp + i * FW, ul, s, sh);
                const uint32_t at = ring_count + i;
                if (alive) alive = fbar_wait(&bar[at % FNS], (at / FNS) & 1u, a.status);
                alive = __all_sync(0xffffffffu, alive);
                const uint8_t *stage = ring + (at % FNS) * FSTAGE;
                float f0 = 0.0f, f1 = 0.0f;
                if (alive) {
                    if (sh) consume_unit_slice<ST>(stage, nbh, s, xq_lane, xsum_tok, g, t, f0, f1);
                    else consume_unit_slice<RT>(stage, nbh, s, xq_lane, xsum_tok, g, t, f0, f1);
                }
                partial[(warp + i * FW) * 32 + lane] = make_float2(f0, f1);
                __syncwarp();
                fproxy_fence();
                if (alive && i + FNS < mine) issue(i + FNS);
            }
            if (alive) ring_count += mine;
            CLOCK(7);
            MARK(1);
            __syncthreads();
            // granules: slices added in order, SwiGLU, digit pairs with one scale per chunk
#pragma unroll 1
            for (uint32_t gl = warp; gl < g1 - g0; gl += FW) {
                const bool sh = gl < n_shg;
                const uint32_t spu = sh ? spu_s : spu_r;
                const uint32_t gi = g0 + gl;                                       // granule over all sources
                const Src sr = sh ? srcs[0] : srcs[1 + (gi - gs) / gr];
                const uint32_t chunk = sh ? gi : (gi - gs) % gr;
                const bool live = t < T && ((sr.mask >> t) & 1u);
                const uint32_t row = sh ? pairs + t : t * k + sr.slot(t);
                float v[4];
                float m = 0.0f;
                bool whole = true;
#pragma unroll
                for (uint32_t u = 0; u < 4; u++) {
                    const uint32_t ul = gl * 4 + u;
                    const uint32_t n0 = sh ? ul * spu_s : n_shu * spu_s + (ul - n_shu) * spu_r;
                    whole &= n0 + spu <= slices;                                   // beyond the partial buffer (never for supported shapes)
                    float f0 = 0.0f, f1 = 0.0f;
#pragma unroll 1
                    for (uint32_t s = 0; s < spu && whole; s++) { const float2 q = partial[(n0 + s) * 32 + lane]; f0 += q.x; f1 += q.y; }
                    const float dx = misc_f[t];
                    const float gate = f0 * dx, upv = f1 * dx;
                    v[u] = live ? gate * fast_sigmoid(gate) * upv : 0.0f;
                    m = fmaxf(m, fabsf(v[u]));
                }
                if (!whole) { if (lane == 0) atomicOr(a.status, QW4SH_ERR_STATE); continue; }
                for (int o = 4; o < 32; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));   // over the eight rows of every unit
                if (live && !finite_f32(m)) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                const bool usable = finite_f32(m) && m > 0.0f;
                const float inv = usable ? __fdividef(127.0f, m) : 0.0f, d = usable ? m * (1.0f / 127.0f) : 0.0f;
                const float4 c = make_float4(d, inv, 254.0f * inv, 0.0f);
                int s1 = 0, s2 = 0;
                uint8_t *out = a.aq + (uint64_t)row * 2u * p.ap + chunk * 32u + g;
#pragma unroll
                for (uint32_t u = 0; u < 4; u++) {
                    uint32_t ra, rb;
                    digit_pair(v[u], c, ra, rb);
                    s1 += (int)(int8_t)(ra & 0xffu); s2 += (int)(int8_t)(rb & 0xffu);
                    if (live) { out[u * 8] = (uint8_t)ra; out[p.ap + u * 8] = (uint8_t)rb; }
                }
                for (int o = 4; o < 32; o <<= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
                if (live && g == 0) a.asc[(uint64_t)row * (imax >> 5) + chunk] = make_float2(d, d * fmaf((float)s2, 1.0f / 254.0f, (float)s1));
            }
        }
        CLOCK(8);
        __threadfence();
        arrive_counter(a.sync + (attempt ? S_ACT1 : S_ACT0));
        if (!wait_counter(a.sync + (attempt ? S_ACT1 : S_ACT0), NS, a.status, misc_u)) return;
        if (attempt == 1) break;
        if (!wait_counter(a.sync + S_ROUTED, T, a.status, misc_u)) return;
        CLOCK(9);
        MARK(2);
        if (fld_acquire(a.sync + S_ROUTE_FAIL)) { leave(); return; }             // a nonfinite logit: y stays untouched
        // ---- the exact routes against the speculation ----
        if (tid < pairs) { ids_x[tid] = __ldcg(a.ids + tid); wts_x[tid] = __ldcg(a.weights + tid); }
        if (tid < T) misc_f[4 + tid] = a.router_mode == 1 ? misc_f[4 + tid] : __ldcg(a.shared_logit + tid);
        __syncthreads();
        bool same = lists_ok;
        if (lists_ok && tid < pairs) same = ((tokmask[ids_x[tid]] >> (tid / k)) & 1u) != 0;   // k distinct ids on both sides: contained = equal
        same = __syncthreads_and(same);
        if (same) {
            if (tid < pairs) { const uint32_t e = ids_x[tid], tok = tid / k; wts_s[tok * k + slotmap[e * 4 + tok]] = wts_x[tid]; }
            __syncthreads();
            break;
        }
        // repair: phase B again with the exact ids (every CTA takes this branch together: same data, same test)
        if (tid < pairs) { ids_s[tid] = ids_x[tid]; wts_s[tid] = wts_x[tid]; }
        if (sc == 0 && tid == 0) atomicAdd(a.sync + S_REPAIRS, 1u);             // repaired launches since the workspace was cleared (diagnostic)
        lists_ok = __syncthreads_and(alive);
    }
    CLOCK(10);

    // ================================ phase C ================================
    if (sc < (H >> 4) && lists_ok) {
        uint8_t *aq = region + p.aq;
        float2 *asc = reinterpret_cast<float2 *>(region + p.asc);
        uint8_t *tiles = region + p.tiles + warp * FNC * FSTAGE;
        float2 *cpartial = reinterpret_cast<float2 *>(region + p.cpartial);
        const uint32_t my_src = n_src > warp ? (n_src - 1 - warp) / FW + 1 : 0;
        const uint32_t n_tiles = ((H >> 4) - sc + NS - 1) / NS;
        const uint32_t steps = my_src * n_tiles;
        uint32_t next_tile = sc, next_src = warp;                              // issues come in step order: the next step's tile and source
        auto issue = [&](uint32_t n) {                                         // this phase has ring barriers of its own, counted from zero
            const uint32_t tile = next_tile, j = next_src;
            next_src += FW;
            if (next_src >= n_src) { next_src = warp; next_tile += NS; }
            const Src s = srcs[j];
            uint8_t *stage = tiles + (n % FNC) * FSTAGE;
            if (s.shared) issue_down_tile<ST>(a.w[6].data, H, IS >> 8, tile * 16, stage, &tilebar[n % FNC], lane);
            else issue_down_tile<RT>(a.w[3].data + (uint64_t)s.expert * a.w[3].expert_bytes, H, I >> 8, tile * 16, stage, &tilebar[n % FNC], lane);
        };
        bool ok = __syncthreads_and(alive);                                    // also: phase B's use of the region is over
        if (ok) {
            asm volatile("fence.proxy.async;" ::: "memory");                      // the digits were written through the generic proxy, by other CTAs
            fproxy_fence();
            const uint32_t aq_bytes = rows_c * 2u * p.ap, asc_bytes = rows_c * (imax >> 5) * 8u;
            if (tid == 0) {
                fbar_expect(abar, aq_bytes + asc_bytes);
                fbulk(aq, a.aq, aq_bytes, abar);
                fbulk(asc, a.asc, asc_bytes, abar);
            }
            for (uint32_t n = 0; n < FNC && n < steps; n++) issue(n);
            ok = __syncthreads_and(fbar_wait(abar, 0, a.status));
        }
        alive = ok;
        CLOCK(11);
        uint32_t n = 0;
#pragma unroll 1
        for (uint32_t ti = 0; ti < n_tiles; ti++) {
            const uint32_t tile = sc + ti * NS;
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 1
            for (uint32_t si = 0; si < my_src; si++, n++) {
                const Src s = srcs[warp + si * FW];
                const uint32_t tokg = g >> 1;
                const uint32_t row_g = s.shared ? pairs + (tokg < T ? tokg : 0) : (((s.mask >> tokg) & 1u) ? tokg * k + s.slot(tokg) : 0);
                const bool live_t = t < T && ((s.mask >> t) & 1u);
                const uint32_t row_t = s.shared ? pairs + (t < T ? t : 0) : (live_t ? t * k + s.slot(t) : 0);
                const uint8_t *aq_lane = aq + (2 * row_g + (g & 1u)) * p.ap + 8 * t;
                const float2 *asc_tok = asc + row_t * (imax >> 5);
                if (alive) alive = fbar_wait(&tilebar[n % FNC], (n / FNC) & 1u, a.status);
                alive = __all_sync(0xffffffffu, alive);
                const uint8_t *stage = tiles + (n % FNC) * FSTAGE;
                float f0 = 0.0f, f1 = 0.0f;
                if (alive) {
                    if (s.shared) consume_down_tile<ST>(stage, IS >> 8, aq_lane, asc_tok, g, t, f0, f1);
                    else consume_down_tile<RT>(stage, I >> 8, aq_lane, asc_tok, g, t, f0, f1);
                }
                __syncwarp();
                fproxy_fence();
                if (alive && n + FNC < steps) issue(n + FNC);
                if (live_t) {
                    const float coef = s.shared ? fast_sigmoid(misc_f[4 + t]) : wts_s[t * k + s.slot(t)];
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
                if (tt < T && alive) {
                    if (!finite_f32(sum)) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.y[(uint64_t)tt * H + tile * 16 + hi * 8 + gg] = sum;
                    if (!hc_add(a.hc, tt, tile * 16 + hi * 8 + gg, H, sum)) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                }
            }
            __syncthreads();
        }
    }
    CLOCK(12);
    MARK(3);
    leave();
#undef CLOCK
#undef MARK
}

}  // namespace qw4

using namespace qw4;

extern "C" int qw4sh_note_launch(const char *name);

static DevTensor fdev(const QW4ShTensor &s) {
    DevTensor t;
    t.data = s.data; t.type = s.type; t.k_storage = s.k_storage; t.k_logical = s.k_logical;
    t.n_out = s.n_out; t.n_experts = s.n_experts; t.row_bytes = s.row_bytes; t.expert_bytes = s.expert_bytes;
    return t;
}

static int g_fused_mode = -1;                          // -1 automatic, 0 never
extern "C" void qw4sh_set_fused_decode(int mode) { g_fused_mode = mode; }
static int g_wrong_speculation = 0;
extern "C" void qw4sh_set_wrong_speculation(int on) { g_wrong_speculation = on ? 1 : 0; }

static bool fused_type(uint32_t type) { return type == T_Q4_K || type == T_IQ2_XXS; }
static uint32_t slice_blocks(uint32_t) { return FGeo<T_Q4_K>::SLICE_BLOCKS; }          // both formats of this path: 512 columns per slice

// Chain CTAs: one per 32 rows of the router (the shared expert's router is row E), and at least
// one per token (chain CTA t routes token t).  The fast mode keeps only the routing CTAs.
static uint32_t chain_ctas(const QW4ShLayer *l, size_t tokens, int router_mode) {
    const uint32_t by_rows = router_mode == 1 ? 0 : (l->experts + 1 + CROWS - 1) / CROWS;
    return by_rows > tokens ? by_rows : (uint32_t)tokens;
}

// Most slices one streaming CTA can get: its share of the granules (whole granules of four units,
// the shared expert's first), each unit cut into its format's number of slices.
static uint32_t partial_capacity(const QW4ShLayer *l, size_t tokens, uint32_t streaming) {
    const uint32_t nbh = l->hidden >> 8, spu_s = nbh / slice_blocks(l->w[4].type), spu_r = nbh / slice_blocks(l->w[1].type);
    const uint64_t total = (l->shared_inter >> 5) + (uint64_t)tokens * l->top_k * (l->inter >> 5);
    const uint32_t per_cta = (uint32_t)((total + streaming - 1) / streaming) + 1;
    return per_cta * 4 * (spu_s > spu_r ? spu_s : spu_r);
}

static FPlan plan_for(const QW4ShLayer *l, size_t tokens, uint32_t streaming) {
    const uint32_t imax = l->inter > l->shared_inter ? l->inter : l->shared_inter;
    return make_fplan(l->hidden, imax, (uint32_t)tokens * l->top_k + (uint32_t)tokens, partial_capacity(l, tokens, streaming));
}

// Bytes of the workspace arrays the kernel needs beyond the common ones (for `cap` tokens, at most FTOK used).
extern "C" void qw4sh_fused_scratch_sizes(const QW4ShLayer *l, size_t *aq_bytes, size_t *asc_bytes, size_t *fast_bytes) {
    const uint32_t imax = l->inter > l->shared_inter ? l->inter : l->shared_inter;
    const size_t rows = (size_t)FTOK * l->top_k + FTOK;
    *aq_bytes = rows * 2 * (imax + 32) + 256;
    *asc_bytes = rows * (imax / 32 + 1) * 8 + 256;
    *fast_bytes = (size_t)FTOK * ((l->experts + 1 + 3) & ~3u) * 4 + 256;
}

// ---- tensor maps of the gate / up matrices ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// The tensor this path streams for resident tensor i: the tensor itself (Q4_K) or its expanded image (IQ2_XXS), whose
// rows have the geometry of Q4_K rows (144 bytes per 256 columns).
static DevTensor fused_view(const QW4ShLayer *l, int i) {
    DevTensor t = fdev(l->w[i]);
    const int holder = (i == 2 || i == 5) ? i - 1 : i;                     // gate and up share the gate's image
    if (t.type == T_IQ2_XXS && l->fused_alt[holder]) {
        t.data = (const uint8_t *)l->fused_alt[holder];
        t.type = T_IQ2N;
        t.row_bytes = (t.k_storage >> 8) * 144u;
        t.expert_bytes = (uint64_t)t.row_bytes * t.n_out;
    }
    return t;
}
// {32-bit words of a row's packed payload, rows of an expert, experts}; box = one slice (288 bytes) of eight rows.
static int rows_map(const DevTensor &t, CUtensorMap *map) {
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess || !fn) return -1;
        encode = (EncodeTiled)fn;
    }
    constexpr uint32_t slice = FGeo<T_Q4_K>::SLICE_BLOCKS * FGeo<T_Q4_K>::BLOCK_BYTES;
    const cuuint64_t dims[3] = {(cuuint64_t)t.row_bytes / 4, t.n_out, t.n_experts};
    const cuuint64_t strides[2] = {(cuuint64_t)t.row_bytes, t.expert_bytes};
    const cuuint32_t box[3] = {slice / 4, 8, 1}, elem[3] = {1, 1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (void *)t.data, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2;
}
static bool fused_type(uint32_t type);
extern "C" void qw4sh_fused_release(QW4ShLayer *l) {
    for (int i = 0; i < 8; i++) { if (l->fused_alt[i]) cudaFree(l->fused_alt[i]); l->fused_alt[i] = nullptr; }
    l->fused_alt_bytes = 0;
    l->fused_maps_ready = 0;
}
// Called once the images are resident.  A layer the path cannot take simply gets no maps and no expanded images; 0
// unless a CUDA call failed.
extern "C" int qw4sh_fused_prepare(QW4ShLayer *l) {
    l->fused_maps_ready = 0;
    l->fused_alt_bytes = 0;
    for (int i = 0; i < 8; i++) l->fused_alt[i] = nullptr;
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    if (g_fused_mode == 0) return 0;                                            // switched off before create: no maps, no expanded images
    if (l->w[2].type != l->w[1].type || l->w[3].type != l->w[1].type || l->w[5].type != l->w[4].type || l->w[6].type != l->w[4].type) return 0;
    for (int i = 1; i <= 6; i++) {
        const QW4ShTensor *t = &l->w[i];
        if (!fused_type(t->type) || t->k_storage % 512 || t->k_logical != t->k_storage || t->n_out % 32 || ((uintptr_t)t->data & 15u) ||
            t->expert_bytes % 16) return 0;
    }
    // expanded images: gate and up of a group share one (unit slices interleaved, held by the gate's slot), down has its own
    for (int i = 1; i <= 6; i++) {
        if (l->w[i].type != T_IQ2_XXS || i == 2 || i == 5) continue;
        const bool pair = i == 1 || i == 4;
        const DevTensor src = fdev(l->w[i]);
        if (pair && (l->w[i + 1].n_out != src.n_out || l->w[i + 1].k_storage != src.k_storage || l->w[i + 1].n_experts != src.n_experts)) return 0;
        const size_t bytes = (size_t)src.n_experts * src.n_out * (src.k_storage >> 9) * 288u * (pair ? 2 : 1);
        cudaError_t e = cudaMalloc(&l->fused_alt[i], bytes);
        if (e == cudaSuccess) e = cudaMemset(l->fused_alt[i], 0, bytes);
        if (e == cudaSuccess) {
            const uint64_t chunks = (uint64_t)src.n_experts * src.n_out * (src.k_storage >> 5);
            iq2_expand_kernel<<<(unsigned)((chunks + 255) / 256), 256>>>(src, (uint8_t *)l->fused_alt[i], pair ? 0 : -1);
            if (pair) iq2_expand_kernel<<<(unsigned)((chunks + 255) / 256), 256>>>(fdev(l->w[i + 1]), (uint8_t *)l->fused_alt[i], 1);
            e = cudaDeviceSynchronize();
        }
        if (e != cudaSuccess) { qw4sh_fused_release(l); return -1; }
        l->fused_alt_bytes += bytes;
    }
    const int which[4] = {1, 2, 4, 5};
    for (int i = 0; i < 4; i++) {
        alignas(64) CUtensorMap map;
        if (rows_map(fused_view(l, which[i]), &map)) { qw4sh_fused_release(l); return -1; }
        memcpy(l->fused_maps[i], &map, sizeof map);
    }
    l->fused_maps_ready = 1;
    return 0;
}

// Probe entry: decode rows of tensor i (1-6) from its expanded image; -3 when the tensor has none.
extern "C" int qw4sh_fused_decode_rows_expanded(const QW4ShLayer *l, int i, size_t expert, size_t row0, size_t rows, float *out, void *stream) {
    if (i < 1 || i > 6 || l->w[i].type != T_IQ2_XXS) return -3;
    const int holder = (i == 2 || i == 5) ? i - 1 : i;
    if (!l->fused_alt[holder]) return -3;
    const int which = i == 3 || i == 6 ? -1 : (i == holder ? 0 : 1);
    const uint64_t total = (uint64_t)rows * l->w[i].k_storage;
    if (!total) return 0;
    iq2n_decode_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t *)l->fused_alt[holder], l->w[i].k_storage,
                                                                                          l->w[i].n_out, (uint32_t)expert, (uint32_t)row0, (uint32_t)rows,
                                                                                          which, out);
    return qw4sh_note_launch("iq2n_decode_rows_kernel");
}

// Whether the one-kernel decode path covers this layer and batch.
extern "C" int qw4sh_fused_supported(const QW4ShLayer *l, size_t tokens, const float *x, const float *y, int grid) {
    if (g_fused_mode == 0 || !l->fused_maps_ready) return 0;
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
    if (I > 512 || IS > 512 || I % 512 || IS % 512) return 0;
    const uint32_t nc = chain_ctas(l, tokens, 0);
    if (grid < 1 || (uint32_t)grid <= nc) return 0;
    const uint32_t streaming = (uint32_t)grid - nc;
    if (streaming * FRMAX < l->experts + 1) return 0;
    if (plan_for(l, tokens, streaming).total > 227u * 1024u || make_cplan(H).total > 227u * 1024u) return 0;
    return 1;
}

template <uint32_t RT, uint32_t ST>
static int launch_fused(const FusedArgs &a, const QW4ShLayer *layer, uint32_t smem, int grid, cudaStream_t stream) {
    static bool configured[64] = {false};                 // per device: the attribute and the residency check
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[device]) {
        e = cudaFuncSetAttribute(fused_decode_kernel<RT, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        if (e != cudaSuccess) return (int)e;
        // the grid barriers need every CTA resident: one per SM, and an SM must take one
        int resident = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fused_decode_kernel<RT, ST>, FT, 227 * 1024 - 1024);
        if (e != cudaSuccess) return (int)e;
        if (resident < 1) return (int)cudaErrorCooperativeLaunchTooLarge;
        configured[device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(FT); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    alignas(64) CUtensorMap maps[4];
    memcpy(maps, layer->fused_maps, sizeof maps);
    e = cudaLaunchKernelEx(&cfg, fused_decode_kernel<RT, ST>, a, maps[0], maps[1], maps[2], maps[3]);
    if (e != cudaSuccess) return (int)e;
    return qw4sh_note_launch("fused_decode_kernel");
}

extern "C" int qw4sh_fused_decode(const QW4ShLayer *layer, const QW4ShWork *work, const float *x, float *y, size_t tokens,
                                  uint32_t *ids_out, float *weights_out, int router_mode, int sm_count) {
    if (!work->fused_aq || !work->fused_asc || !work->logits_fast) return -5;
    FusedArgs a;
    for (int i = 0; i < 8; i++) a.w[i] = fused_view(layer, i);
    a.x = x; a.y = y;
    a.hc = HcAdd{work->hc_residual, work->hc_inject, work->hc_streams};
    a.status_mirror = work->status_mirror;
    a.tokens = (uint32_t)tokens; a.hidden = layer->hidden; a.experts = layer->experts; a.top_k = layer->top_k;
    a.inter = layer->inter; a.shared_inter = layer->shared_inter; a.norm = layer->norm; a.router_mode = router_mode == 0 && g_wrong_speculation ? 2 : router_mode;
    a.logits = work->logits; a.shared_logit = work->shared_logit; a.ids = work->ids; a.weights = work->weights;
    a.logits_fast = work->logits_fast; a.fast_pitch = (layer->experts + 1 + 3) & ~3u;
    a.aq = (uint8_t *)work->fused_aq; a.asc = (float2 *)work->fused_asc;
    a.ids_out = ids_out; a.weights_out = weights_out;
    a.sync = work->sync; a.status = work->status;
    const uint32_t rt = layer->w[1].type, st = layer->w[4].type;
    const uint32_t streaming = (uint32_t)sm_count - chain_ctas(layer, tokens, 0);     // the same split in every mode (plans, capacity)
    a.chain_ctas = (uint32_t)sm_count - streaming;
    a.partial_slices = partial_capacity(layer, tokens, streaming);
    const FPlan p = plan_for(layer, tokens, streaming);
    const CPlan c = make_cplan(layer->hidden);
    const uint32_t smem = p.total > c.total ? p.total : c.total;
    if (smem > 227u * 1024u - 1024u) return -4;
    cudaStream_t s = (cudaStream_t)work->stream;
    if (rt == T_Q4_K) return st == T_Q4_K ? launch_fused<T_Q4_K, T_Q4_K>(a, layer, smem, sm_count, s) : launch_fused<T_Q4_K, T_IQ2N>(a, layer, smem, sm_count, s);
    return st == T_Q4_K ? launch_fused<T_IQ2N, T_Q4_K>(a, layer, smem, sm_count, s) : launch_fused<T_IQ2N, T_IQ2N>(a, layer, smem, sm_count, s);
}
