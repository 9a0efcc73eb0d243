// Expert products for prefill-sized groups on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with TMEM accumulators, packed weight tiles staged by 2-D TMA.
//
// Q4_K weights are w = d * (sc * q) - dmin * m with q a 4-bit code, sc / m 6-bit integers per
// 32 columns and d / dmin fp16 per 256 columns (picoforge src/qwen4_packed.c:86-93).  sc * q
// (<= 945) and m (<= 63) are exact in fp16, so the tensor cores multiply EXACT integers:
//
//   A   128 weight rows x K of (sc * q) as fp16, produced from the packed bytes by the
//       dequantising warps (two half-precision operations per two weights),
//   B   up to 32 token rows x K of the activation, split into fp16 hi + lo (x = hi + lo to about
//       22 bits): the 32 hi rows and the 32 lo rows are the MMA's 64 columns, so A is read once,
//   min term: a second, K = 16 product per 256-column block of the block's eight m values with
//       the activations' eight 32-column sums (also hi + lo),
//
// and the fp16 super-scales are applied in FP32 when the block's accumulators are read back:
// acc += d * Q - dmin * M.  The result differs from the FP32 reference only by the activation
// split (2^-22 relative), far inside the layer's 1e-3 bound.
//
// Weights sit on the MMA's M axis (128 rows), tokens on N (32): an expert's rows are cut into
// groups of <= 32 (dispatch order, so per-expert lists stay the reference's), and a work item is
// (group, tile of 128 weight rows).  CTAs are persistent and walk the item list with a stride.
//
// Warp roles in a CTA (15 warps):
//   0-3    epilogue: one TMEM lane (= weight row) per thread; per 256-column block read Q and M
//          with tcgen05.ld, scale, accumulate; at the end SwiGLU (gate/up) or a plain store (down).
//          gate/up writes the activation directly as the down product's B operand (fp16 hi/lo,
//          32-column sums), so no separate conversion pass runs in between.
//   4-11   dequantise: packed block rows (shared memory, from TMA) -> fp16 operand tiles, K-major rows of
//          128 bytes (64 columns) with the 128-byte swizzle the tensor cores read at full rate.
//   12     TMA producer: one 2-D tensor copy (128 rows x 144 bytes) per matrix and block.
//   13     MMA issuer: one elected lane issues tcgen05.mma / tcgen05.commit.
//   14     activation loader: 16-byte cp.async gathers of the group's token rows.
//
// Every mbarrier wait is bounded (about a second); a role that gives up records QW4SH_ERR_STATE
// and all roles leave their loops; TMEM is freed on every path.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "cuda_shim.h"
#include "formats.cuh"

namespace qw4 {

constexpr int PT_EPI = 4, PT_DEQ = 8;                       // warps
constexpr int PT_WARPS = PT_EPI + PT_DEQ + 3, PT_THREADS = PT_WARPS * 32;
constexpr int PT_W_TMA = PT_EPI + PT_DEQ, PT_W_MMA = PT_W_TMA + 1, PT_W_ACT = PT_W_TMA + 2;
constexpr uint32_t PT_ROWS = 128;                           // weight rows per item (MMA M)
constexpr uint32_t PT_TOK = 32;                             // token rows per group (MMA N)
constexpr uint32_t PT_KS = 64;                              // columns per operand stage
constexpr uint32_t PT_STAGES = 2;                           // weight operand stages
constexpr uint32_t PT_BSTAGES = 8;                          // activation operand stages (deep: their latency is a cache round trip)
constexpr uint32_t PT_BLOCK = 144;                          // Q4_K block bytes
constexpr uint32_t PT_N = 2 * PT_TOK;                        // MMA N: the tokens' hi halves, then their lo halves
constexpr uint32_t PT_TMEM_COLS = 512;                      // 2 buffers x (Q gate, M gate, Q up, M up) x 64

// Shared-memory map (bytes).
constexpr uint32_t PT_BARS = 0;                             // mbarriers
constexpr uint32_t PT_TMEMPTR = 1024;
constexpr uint32_t PT_DSC = 2048;                           // [2][2][128] (d, dmin) words
constexpr uint32_t PT_PK = 4096;                            // [2][2][128 x 144]; the operand tiles behind it start on a 1024-byte boundary
constexpr uint32_t PT_PK_ONE = PT_ROWS * PT_BLOCK;          // 18432
constexpr uint32_t PT_A = PT_PK + 2 * 2 * PT_PK_ONE;        // [stages][2][128 rows][128 bytes], 128-byte swizzle
static_assert(PT_A % 1024 == 0, "swizzled operand tiles need 1024-byte alignment");
constexpr uint32_t PT_A_ONE = 8 * PT_ROWS * 16;             // 16384
constexpr uint32_t PT_B = PT_A + PT_STAGES * 2 * PT_A_ONE;  // [b stages][64 rows][128 bytes], 128-byte swizzle: row n < 32 hi of token n, else lo of token n - 32
constexpr uint32_t PT_B_ONE = 8 * PT_TOK * 16;              // 4096: half a stage
constexpr uint32_t PT_AM = PT_B + PT_BSTAGES * 2 * PT_B_ONE; // [2][2][2][128][16]
constexpr uint32_t PT_AM_ONE = 2 * PT_ROWS * 16;            // 4096
constexpr uint32_t PT_BS = PT_AM + 2 * 2 * PT_AM_ONE;       // [2][2][64][16]
constexpr uint32_t PT_BS_ONE = 2 * PT_TOK * 16;             // 1024: half a buffer
constexpr uint32_t PT_SMEM = PT_BS + 2 * 2 * PT_BS_ONE;

// Column order inside a group of eight (an involution): what the nibble extraction yields.
__host__ __device__ __forceinline__ uint32_t pt_perm(uint32_t j) { return (j & ~7u) | ((0x75643120u >> (4 * (j & 7u))) & 7u); }

struct PGroup { uint32_t expert, first, count, pad; };

struct PrefillArgs {
    uint32_t mode;                      // 0 gate/up + SwiGLU, 1 down
    uint32_t k;                         // reduction length (multiple of 256)
    uint32_t n_out;                     // weight rows per expert (multiple of 128)
    uint32_t k_div;                     // gate/up: input row = pair / k_div
    const PGroup *groups;
    const uint32_t *n_groups;
    const uint32_t *row_to_pair;        // nullptr: pair = row (shared expert)
    const __half *in_hi, *in_lo;        // [rows][k], permuted columns
    const __half *sum_hi, *sum_lo;      // [rows][k / 32]
    __half *out_hi, *out_lo;            // gate/up: [pairs][n_out] permuted; sums below
    __half *osum_hi, *osum_lo;          // [pairs][n_out / 32]
    float *out;                         // gate/up: act [pairs][n_out] (may be nullptr); down: out [pairs][n_out]
    uint32_t *status;
    unsigned long long *debug;          // optional [64]: cycles CTA 0's roles spent in their waits (profiling aid)
};

// ---- PTX helpers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ps_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ps_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void pbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ps_u32(bar)) : "memory");
}
__device__ __forceinline__ void pbar_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ps_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool pbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(ps_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; `dead` (shared memory) is set by whoever gives up, and ends every other wait.
__device__ __noinline__ bool pbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *dead, uint32_t *status) {
    if (pbar_try(bar, parity)) return true;
    const long long start = clock64();
    while (!pbar_try(bar, parity)) {
        if (*dead) return false;
        if (clock64() - start > (1ll << 31)) { *dead = 1; atomicOr(status, QW4SH_ERR_STATE); return false; }
    }
    return true;
}
// Wait with the time spent added to a role-local counter.
#define PT_WAIT(counter, bar, parity) ([&]() { const long long t0_ = clock64(); const bool ok_ = pbar_wait(bar, parity, dead, a.status); counter += clock64() - t0_; return ok_; }())

__device__ __forceinline__ void ptma_2d(void *dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(ps_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(ps_u32(bar)) : "memory");
}
__device__ __forceinline__ void pcp_async16(void *dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(ps_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void pcp_async_arrive(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(ps_u32(bar)) : "memory");
}
__device__ __forceinline__ void pfence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void ptc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ptc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ptc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ps_u32(bar)) : "memory");
}
__device__ __forceinline__ void ptc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ptc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Shared-memory matrix descriptor: no swizzle, K-major; lbo = bytes between the two 8-column core
// matrices of one MMA, sbo = bytes between 8-row groups; descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t pdesc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) |
           (1ull << 46);
}
// Shared-memory matrix descriptor of a K-major tile of 128-byte rows with the 128-byte swizzle (the
// 16-byte piece c of row r sits at piece c ^ (r & 7)); 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t pdesc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D = F32, A = B = F16, both K-major, N = 64, M = 128.
constexpr uint32_t PT_IDESC = (1u << 4) | ((PT_N >> 3) << 17) | ((PT_ROWS >> 4) << 24);

// Q4_K scale / min bytes of sub-blocks 2c and 2c + 1 from the three header words (bytes 4..15).
__device__ __forceinline__ void pt_scale_min(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t sub, uint32_t &sc, uint32_t &mn) {
    const uint32_t lo_s = (w0 >> (8 * (sub & 3u))) & 0xffu, lo_m = (w1 >> (8 * (sub & 3u))) & 0xffu, hi = (w2 >> (8 * (sub & 3u))) & 0xffu;
    if (sub < 4) { sc = lo_s & 63u; mn = lo_m & 63u; }
    else { sc = (hi & 15u) | ((lo_s & 192u) >> 2); mn = (hi >> 4) | ((lo_m & 192u) >> 2); }
}

template <int MODE>
__global__ void __launch_bounds__(PT_THREADS, 1) prefill_tc_kernel(const __grid_constant__ CUtensorMap map0,
                                                                    const __grid_constant__ CUtensorMap map1, const PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr uint32_t MATS = MODE == 0 ? 2 : 1;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + PT_BARS);
    uint64_t *pk_full = bars, *pk_empty = bars + 2, *acc_full = bars + 4, *acc_empty = bars + 6, *a_full = bars + 8,
             *a_empty = a_full + PT_STAGES, *b_full = a_empty + PT_STAGES, *b_empty = b_full + PT_BSTAGES;
    volatile uint32_t *dead = reinterpret_cast<volatile uint32_t *>(smem + PT_TMEMPTR + 8);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + PT_TMEMPTR);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t nb = a.k >> 8, tiles = a.n_out / PT_ROWS;
    long long w0 = 0, w1 = 0, w2 = 0;                                     // cycles in this thread's waits, by kind
    const long long t_begin = clock64();

    if (tid == 0) {
        for (int i = 0; i < 2; i++) { pbar_init(&pk_full[i], 1); pbar_init(&pk_empty[i], PT_DEQ); pbar_init(&acc_full[i], 1); pbar_init(&acc_empty[i], PT_EPI); }
        for (uint32_t i = 0; i < PT_STAGES; i++) { pbar_init(&a_full[i], PT_DEQ); pbar_init(&a_empty[i], 1); }
        for (uint32_t i = 0; i < PT_BSTAGES; i++) { pbar_init(&b_full[i], 32); pbar_init(&b_empty[i], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *dead = 0;
    }
    // the second core-matrix column of the min operands stays zero
    for (uint32_t i = tid; i < 2 * 2 * PT_AM_ONE / 16; i += PT_THREADS) reinterpret_cast<uint4 *>(smem + PT_AM)[i] = make_uint4(0, 0, 0, 0);
    for (uint32_t i = tid; i < 2 * 2 * PT_BS_ONE / 16; i += PT_THREADS) reinterpret_cast<uint4 *>(smem + PT_BS)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ps_u32(tmem_slot)), "r"(PT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pfence_async();
    ptc_fence_before();
    __syncthreads();
    ptc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t n_groups = *a.n_groups;
    const uint32_t n_items = n_groups * tiles;

    if (warp == PT_W_TMA) {
        // ---------------- packed weight blocks by TMA ----------------
        uint32_t blk = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            const PGroup grp = a.groups[it / tiles];
            const uint32_t row0 = grp.expert * a.n_out + (it % tiles) * PT_ROWS;
            for (uint32_t b = 0; b < nb && ok; b++, blk++) {
                const uint32_t pb = blk & 1u;
                if (blk >= 2) ok = PT_WAIT(w0, &pk_empty[pb], ((blk >> 1) - 1) & 1u);
                if (!ok) break;
                if (lane == 0) {
                    pbar_expect(&pk_full[pb], MATS * PT_PK_ONE);
                    ptma_2d(smem + PT_PK + (pb * 2 + 0) * PT_PK_ONE, &map0, b * PT_BLOCK, row0, &pk_full[pb]);
                    if (MODE == 0) ptma_2d(smem + PT_PK + (pb * 2 + 1) * PT_PK_ONE, &map1, b * PT_BLOCK, row0, &pk_full[pb]);
                }
                __syncwarp();
            }
        }
        // leave only when the copies issued last have landed (or the wait ran out)
        if (blk >= 1) pbar_wait(&pk_full[(blk - 1) & 1u], ((blk - 1) >> 1) & 1u, dead, a.status);
        if (blk >= 2) pbar_wait(&pk_full[(blk - 2) & 1u], ((blk - 2) >> 1) & 1u, dead, a.status);
    } else if (warp == PT_W_ACT) {
        // ---------------- activation rows: fp16 hi / lo and 32-column sums ----------------
        uint32_t st = 0, blk = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            const PGroup grp = a.groups[it / tiles];
            uint32_t src_row = 0;
            if (lane < grp.count) {
                const uint32_t pair = a.row_to_pair ? a.row_to_pair[grp.first + lane] : grp.first + lane;
                src_row = pair / a.k_div;
            }
            const uint32_t bytes = lane < grp.count ? 16u : 0u;               // rows beyond the group read as zero
            for (uint32_t b = 0; b < nb && ok; b++, blk++) {
                for (uint32_t c = 0; c < 4 && ok; c++, st++) {
                    const uint32_t slot = st % PT_BSTAGES;
                    if (st >= PT_BSTAGES) ok = PT_WAIT(w0, &b_empty[slot], (st / PT_BSTAGES - 1) & 1u);
                    if (!ok) break;
                    const uint32_t col0 = b * 256 + c * PT_KS;
                    uint8_t *dst = smem + PT_B + slot * 2 * PT_B_ONE;
                    // lane = token row; eight 16-byte pieces of hi and of lo
#pragma unroll
                    for (uint32_t k8 = 0; k8 < 8; k8++) {
                        pcp_async16(dst + lane * 128 + ((k8 ^ (lane & 7u)) << 4), a.in_hi + (uint64_t)src_row * a.k + col0 + k8 * 8, bytes);
                        pcp_async16(dst + (PT_TOK + lane) * 128 + ((k8 ^ (lane & 7u)) << 4), a.in_lo + (uint64_t)src_row * a.k + col0 + k8 * 8, bytes);
                    }
                    if (c == 0) {                                                // the block's eight 32-column sums
                        uint8_t *sd = smem + PT_BS + (blk & 1u) * 2 * PT_BS_ONE;
                        pcp_async16(sd + lane * 16, a.sum_hi + (uint64_t)src_row * (a.k >> 5) + b * 8, bytes);
                        pcp_async16(sd + (PT_TOK + lane) * 16, a.sum_lo + (uint64_t)src_row * (a.k >> 5) + b * 8, bytes);
                    }
                    pcp_async_arrive(&b_full[slot]);
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == PT_W_MMA) {
        // ---------------- tcgen05.mma issue ----------------
        uint32_t st = 0, blk = 0;
        bool ok = true;
        // operand descriptors: slot / buffer / k-step offsets are added to the 16-byte address field
        const uint64_t a_desc0 = pdesc_sw128(ps_u32(smem + PT_A)), b_desc0 = pdesc_sw128(ps_u32(smem + PT_B));
        const uint64_t am_desc0 = pdesc(ps_u32(smem + PT_AM), PT_ROWS * 16, 128), bs_desc0 = pdesc(ps_u32(smem + PT_BS), PT_N * 16, 128);
        for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            for (uint32_t b = 0; b < nb && ok; b++, blk++) {
                const uint32_t p = blk & 1u;
                if (blk >= 2) ok = PT_WAIT(w2, &acc_empty[p], ((blk >> 1) - 1) & 1u);
                for (uint32_t c = 0; c < 4 && ok; c++, st++) {
                    const uint32_t slot = st % PT_STAGES, bslot = st % PT_BSTAGES;
                    ok = PT_WAIT(w0, &a_full[slot], (st / PT_STAGES) & 1u);
                    if (ok) ok = PT_WAIT(w1, &b_full[bslot], (st / PT_BSTAGES) & 1u);
                    if (!ok) break;
                    pfence_async();
                    ptc_fence_after();
                    if (lane == 0) {
                        const uint32_t acc = tmem_base + p * 256;
#pragma unroll
                        for (uint32_t j = 0; j < PT_KS / 16; j++) {
                            const uint64_t bd = b_desc0 + bslot * ((2 * PT_B_ONE) >> 4) + j * 2;       // 32 bytes (16 columns) along the row per k-step
#pragma unroll
                            for (uint32_t m = 0; m < MATS; m++)
                                ptc_mma_f16(acc + m * 128, a_desc0 + (slot * 2 + m) * (PT_A_ONE >> 4) + j * 2, bd, PT_IDESC,
                                            (c | j) ? 1u : 0u);
                        }
                        if (c == 0) {                                            // min term of this block
#pragma unroll
                            for (uint32_t m = 0; m < MATS; m++)
                                ptc_mma_f16(acc + m * 128 + 64, am_desc0 + (p * 2 + m) * (PT_AM_ONE >> 4), bs_desc0 + p * ((2 * PT_BS_ONE) >> 4), PT_IDESC, 0u);
                        }
                        ptc_commit(&a_empty[slot]);
                        ptc_commit(&b_empty[bslot]);
                        if (c == 3) ptc_commit(&acc_full[p]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp >= PT_EPI) {
        // ---------------- dequantise: packed bytes -> fp16 (sc * q) operand tiles ----------------
        // a warp owns 16 rows: lanes (l & 7) + 8 (l >> 4) pick the row, bit 3 of the lane one of two 8-byte pieces, so a
        // half-warp's 64-bit reads of the 144-byte-pitch rows fall in distinct banks
        const uint32_t dw = warp - PT_EPI, row = dw * 16 + (lane & 7u) + ((lane >> 4) << 3), isel = (lane >> 3) & 1u;
        uint32_t st = 0, blk = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            for (uint32_t b = 0; b < nb && ok; b++, blk++) {
                const uint32_t pb = blk & 1u;
                ok = PT_WAIT(w0, &pk_full[pb], (blk >> 1) & 1u);
                if (ok && blk >= 2) ok = PT_WAIT(w1, &acc_empty[pb], ((blk >> 1) - 1) & 1u);   // scales / min operands of block - 2 are read
                if (!ok) break;
                uint32_t hdr[MATS][4];
#pragma unroll
                for (uint32_t m = 0; m < MATS; m++) {
                    const uint4 h = *reinterpret_cast<const uint4 *>(smem + PT_PK + (pb * 2 + m) * PT_PK_ONE + row * PT_BLOCK);
                    hdr[m][0] = h.x; hdr[m][1] = h.y; hdr[m][2] = h.z; hdr[m][3] = h.w;
                }
                if (isel == 0) {                                                 // scales and min operand, once per row and block
#pragma unroll
                    for (uint32_t m = 0; m < MATS; m++) {
                        reinterpret_cast<uint32_t *>(smem + PT_DSC)[(pb * 2 + m) * 128 + row] = hdr[m][0];
                        uint32_t mins[4];
#pragma unroll
                        for (uint32_t q = 0; q < 4; q++) {
                            uint32_t s0, m0, s1, m1;
                            pt_scale_min(hdr[m][1], hdr[m][2], hdr[m][3], 2 * q, s0, m0);
                            pt_scale_min(hdr[m][1], hdr[m][2], hdr[m][3], 2 * q + 1, s1, m1);
                            const __half2 v = __halves2half2(__ushort2half_rn((unsigned short)m0), __ushort2half_rn((unsigned short)m1));
                            mins[q] = *reinterpret_cast<const uint32_t *>(&v);
                        }
                        *reinterpret_cast<uint4 *>(smem + PT_AM + (pb * 2 + m) * PT_AM_ONE + row * 16) = make_uint4(mins[0], mins[1], mins[2], mins[3]);
                    }
                }
                for (uint32_t c = 0; c < 4 && ok; c++, st++) {
                    const uint32_t slot = st % PT_STAGES;
                    if (st >= PT_STAGES) ok = PT_WAIT(w2, &a_empty[slot], (st / PT_STAGES - 1) & 1u);
                    if (!ok) break;
#pragma unroll
                    for (uint32_t m = 0; m < MATS; m++) {
                        uint32_t sc_lo, sc_hi, unused;
                        pt_scale_min(hdr[m][1], hdr[m][2], hdr[m][3], 2 * c, sc_lo, unused);
                        pt_scale_min(hdr[m][1], hdr[m][2], hdr[m][3], 2 * c + 1, sc_hi, unused);
                        const __half2 s_lo = __half2half2(__ushort2half_rn((unsigned short)sc_lo)), s_hi = __half2half2(__ushort2half_rn((unsigned short)sc_hi));
                        const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
                        const uint8_t *qs = smem + PT_PK + (pb * 2 + m) * PT_PK_ONE + row * PT_BLOCK + 16 + c * 32;
                        uint8_t *dst = smem + PT_A + (slot * 2 + m) * PT_A_ONE + row * 128;
#pragma unroll
                        for (uint32_t ii = 0; ii < 2; ii++) {
                            const uint32_t i = ii * 2 + isel;                    // bytes 8i..8i+7: columns 8i.. (low nibbles) and 32 + 8i.. (high)
                            const uint2 q = *reinterpret_cast<const uint2 *>(qs + 8 * i);
                            uint32_t lo[4], hi[4];
                            const uint32_t w[2] = {q.x, q.y};
#pragma unroll
                            for (int h = 0; h < 2; h++) {
                                // (byte0, byte2) and (byte1, byte3) of the word as half2 1024 + nibble
                                const uint32_t l0 = (w[h] & 0x000f000fu) | 0x64006400u, l1 = ((w[h] >> 8) & 0x000f000fu) | 0x64006400u;
                                const uint32_t h0 = ((w[h] >> 4) & 0x000f000fu) | 0x64006400u, h1 = ((w[h] >> 12) & 0x000f000fu) | 0x64006400u;
                                const __half2 a0 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&l0), k1024), s_lo);
                                const __half2 a1 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&l1), k1024), s_lo);
                                const __half2 b0 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&h0), k1024), s_hi);
                                const __half2 b1 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&h1), k1024), s_hi);
                                lo[2 * h] = *reinterpret_cast<const uint32_t *>(&a0); lo[2 * h + 1] = *reinterpret_cast<const uint32_t *>(&a1);
                                hi[2 * h] = *reinterpret_cast<const uint32_t *>(&b0); hi[2 * h + 1] = *reinterpret_cast<const uint32_t *>(&b1);
                            }
                            *reinterpret_cast<uint4 *>(dst + ((i ^ (row & 7u)) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                            *reinterpret_cast<uint4 *>(dst + (((4 + i) ^ (row & 7u)) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        }
                    }
                    pfence_async();
                    __syncwarp();
                    if (lane == 0) pbar_arrive(&a_full[slot]);
                }
                __syncwarp();
                if (ok && lane == 0) pbar_arrive(&pk_empty[pb]);
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> scales -> SwiGLU / store ----------------
        const uint32_t row = warp * 32 + lane;                                   // TMEM lane = weight row inside the tile
        const uint32_t lane_base = (warp * 32) << 16;
        uint32_t blk = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            const PGroup grp = a.groups[it / tiles];
            const uint32_t tile = it % tiles;
            float acc[MATS][PT_TOK];
#pragma unroll
            for (uint32_t m = 0; m < MATS; m++)
#pragma unroll
                for (uint32_t n = 0; n < PT_TOK; n++) acc[m][n] = 0.0f;
            for (uint32_t b = 0; b < nb && ok; b++, blk++) {
                const uint32_t p = blk & 1u;
                ok = PT_WAIT(w0, &acc_full[p], (blk >> 1) & 1u);
                if (!ok) break;
                ptc_fence_after();
#pragma unroll
                for (uint32_t m = 0; m < MATS; m++) {
                    const uint32_t dd = reinterpret_cast<const uint32_t *>(smem + PT_DSC)[(p * 2 + m) * 128 + row];
                    const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xffffu))), dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
                    uint32_t v[32];
#pragma unroll
                    for (uint32_t part = 0; part < 2; part++) {                  // hi and lo halves of the activation
                        ptc_ld32(tmem_base + lane_base + p * 256 + m * 128 + part * 32, v);
#pragma unroll
                        for (uint32_t n = 0; n < PT_TOK; n++) acc[m][n] = fmaf(d, __uint_as_float(v[n]), acc[m][n]);
                        ptc_ld32(tmem_base + lane_base + p * 256 + m * 128 + 64 + part * 32, v);
#pragma unroll
                        for (uint32_t n = 0; n < PT_TOK; n++) acc[m][n] = fmaf(-dmin, __uint_as_float(v[n]), acc[m][n]);
                    }
                }
                ptc_fence_before();
                __syncwarp();
                if (lane == 0) pbar_arrive(&acc_empty[p]);
            }
            if (!ok) break;
            const uint32_t col = tile * PT_ROWS + row;                           // output column of this thread
            const uint32_t my_pair = lane < grp.count ? (a.row_to_pair ? a.row_to_pair[grp.first + lane] : grp.first + lane) : 0;
#pragma unroll
            for (uint32_t n = 0; n < PT_TOK; n++) {
                const bool live = n < grp.count;                                 // warp-uniform
                const uint32_t pair = __shfl_sync(0xffffffffu, my_pair, n);
                if (MODE == 0) {
                    const float g = acc[0][n], u = acc[MATS - 1][n];
                    const float e = __expf(-fabsf(g));
                    const float sig = g >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
                    const float v = g * sig * u;
                    const __half vh = __float2half_rn(v), vl = __float2half_rn(v - __half2float(vh));
                    float s = v;                                                 // sum over the warp's 32 columns: one 32-column chunk
                    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (live) {
                        if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                        a.out_hi[(uint64_t)pair * a.n_out + pt_perm(col)] = vh;
                        a.out_lo[(uint64_t)pair * a.n_out + pt_perm(col)] = vl;
                        if (a.out) a.out[(uint64_t)pair * a.n_out + col] = v;
                        if (lane == 0) {
                            const __half sh = __float2half_rn(s);
                            a.osum_hi[(uint64_t)pair * (a.n_out >> 5) + (col >> 5)] = sh;
                            a.osum_lo[(uint64_t)pair * (a.n_out >> 5) + (col >> 5)] = __float2half_rn(s - __half2float(sh));
                        }
                    }
                } else if (live) {
                    const float v = acc[0][n];
                    if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) atomicOr(a.status, QW4SH_ERR_NONFINITE);
                    a.out[(uint64_t)pair * a.n_out + col] = v;
                }
            }
        }
    }
    if (a.debug && blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == PT_EPI || warp >= PT_W_TMA)) {
        const uint32_t role = warp == 0 ? 0 : warp == PT_EPI ? 1 : 2 + (warp - PT_W_TMA);
        a.debug[role * 4] = (unsigned long long)w0; a.debug[role * 4 + 1] = (unsigned long long)w1;
        a.debug[role * 4 + 2] = (unsigned long long)w2; a.debug[role * 4 + 3] = (unsigned long long)(clock64() - t_begin);
    }
    // ---------------- teardown: TMEM is freed on every path ----------------
    ptc_fence_before();
    __syncthreads();
    if (warp == 0) {
        ptc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PT_TMEM_COLS) : "memory");
    }
}

// x [rows][k] -> fp16 hi / lo (columns permuted inside groups of eight) and 32-column sums hi / lo.
// One warp per 32-column chunk.
__global__ void __launch_bounds__(256) split_rows_kernel(const float *__restrict__ x, uint32_t rows, uint32_t k, __half *hi, __half *lo,
                                                         __half *sum_hi, __half *sum_lo) {
    const uint32_t chunks = k >> 5, lane = threadIdx.x & 31u;
    for (uint64_t w = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5); w < (uint64_t)rows * chunks; w += (uint64_t)gridDim.x * 8) {
        const uint32_t r = (uint32_t)(w / chunks), c = (uint32_t)(w % chunks), col = c * 32 + lane;
        const float v = x[(uint64_t)r * k + col];
        const __half h = __float2half_rn(v), l = __float2half_rn(v - __half2float(h));
        hi[(uint64_t)r * k + pt_perm(col)] = h;
        lo[(uint64_t)r * k + pt_perm(col)] = l;
        float s = v;
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            const __half sh = __float2half_rn(s);
            sum_hi[(uint64_t)r * chunks + c] = sh;
            sum_lo[(uint64_t)r * chunks + c] = __float2half_rn(s - __half2float(sh));
        }
    }
}

// Groups of at most 32 rows out of the expert-sorted lists: one CTA, thread i owns active expert i (then i + 1024,
// ...), a block-wide exclusive scan of the group counts gives every expert its place in the list.  The order is
// the serial one: active experts in ascending order, each expert's groups by ascending row.
__global__ void __launch_bounds__(1024) build_groups32_kernel(const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ active,
                                                              PGroup *groups, uint32_t *n_groups) {
    __shared__ uint32_t wsum[32];
    __shared__ uint32_t s_base;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, n_active = active[0];
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (uint32_t i0 = 0; i0 < n_active; i0 += 1024) {
        const uint32_t i = i0 + tid;
        uint32_t e = 0, first = 0, end = 0;
        if (i < n_active) { e = active[1 + i]; first = offsets[e]; end = offsets[e + 1]; }
        const uint32_t count = (end - first + PT_TOK - 1) / PT_TOK;
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
        for (uint32_t r = first; r < end; r += PT_TOK) groups[at++] = PGroup{e, r, min(PT_TOK, end - r), 0};
        __syncthreads();
        if (tid == 1023) s_base = at;                                // inclusive end of the last thread = end of this pass
        __syncthreads();
    }
    if (tid == 0) *n_groups = s_base;
}
__global__ void build_dense_groups32_kernel(uint32_t tokens, PGroup *groups, uint32_t *n_groups) {
    const uint32_t n = (tokens + PT_TOK - 1) / PT_TOK;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        groups[i] = PGroup{0, i * PT_TOK, min(PT_TOK, tokens - i * PT_TOK), 0};
    if (blockIdx.x == 0 && threadIdx.x == 0) *n_groups = n;
}

}  // namespace qw4

using namespace qw4;

extern "C" int qw4sh_note_launch(const char *name);

// ---- tensor maps --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiled g_encode = nullptr;
static int encode_entry() {
    if (g_encode) return 0;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess || !fn) return -1;
    g_encode = (EncodeTiled)fn;
    return 0;
}
// All rows of all experts of a Q4_K tensor as a [rows][row bytes] byte matrix; box = 128 rows x one block.
static int make_map(const QW4ShTensor *t, CUtensorMap *map) {
    if (encode_entry()) return -1;
    const cuuint64_t dims[2] = {(cuuint64_t)t->row_bytes, (cuuint64_t)t->n_out * t->n_experts};
    const cuuint64_t strides[1] = {(cuuint64_t)t->row_bytes};
    const cuuint32_t box[2] = {PT_BLOCK, PT_ROWS}, elem[2] = {1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)t->data, dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2;
}

static unsigned long long *g_prefill_debug = nullptr;
extern "C" void qw4sh_prefill_debug(void *words) { g_prefill_debug = (unsigned long long *)words; }

extern "C" int qw4sh_prefill_supported(const QW4ShTensor *w, int mode) {
    if (w->type != T_Q4_K) return 0;
    if (w->k_storage % 256 || w->k_logical != w->k_storage || w->n_out % PT_ROWS) return 0;
    if ((uintptr_t)w->data & 15u || w->row_bytes % 16) return 0;
    (void)mode;
    return 1;
}

extern "C" int qw4sh_split_rows(const float *x, uint32_t rows, uint32_t k, void *hi, void *lo, void *sum_hi, void *sum_lo, void *stream) {
    if (!rows) return 0;
    const uint64_t warps = (uint64_t)rows * (k >> 5);
    const unsigned blocks = (unsigned)((warps + 7) / 8 > 4736 ? 4736 : (warps + 7) / 8);
    split_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, rows, k, (__half *)hi, (__half *)lo, (__half *)sum_hi, (__half *)sum_lo);
    return qw4sh_note_launch("split_rows_kernel");
}
extern "C" int qw4sh_build_groups32(const uint32_t *offsets, const uint32_t *active, void *groups, uint32_t *n_groups, void *stream) {
    build_groups32_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(offsets, active, (PGroup *)groups, n_groups);
    return qw4sh_note_launch("build_groups32_kernel");
}
extern "C" int qw4sh_build_dense_groups32(uint32_t tokens, void *groups, uint32_t *n_groups, void *stream) {
    build_dense_groups32_kernel<<<(tokens / PT_TOK + 256) / 256, 256, 0, (cudaStream_t)stream>>>(tokens, (PGroup *)groups, n_groups);
    return qw4sh_note_launch("build_dense_groups32_kernel");
}

// mode 0: gate (w0) + up (w1) + SwiGLU; mode 1: down (w0).  Inputs are the split rows of
// qw4sh_split_rows (or of a mode-0 launch); see PrefillArgs for the outputs.
extern "C" int qw4sh_prefill_tc(int mode, const QW4ShTensor *w0, const QW4ShTensor *w1, const void *groups, const uint32_t *n_groups,
                                const uint32_t *row_to_pair, uint32_t k_div, const void *in_hi, const void *in_lo, const void *sum_hi,
                                const void *sum_lo, void *out_hi, void *out_lo, void *osum_hi, void *osum_lo, float *out, uint32_t *status,
                                int ctas, void *stream) {
    CUtensorMap m0, m1;
    if (make_map(w0, &m0) || make_map(w1 ? w1 : w0, &m1)) return -6;
    PrefillArgs a;
    a.mode = (uint32_t)mode; a.k = w0->k_storage; a.n_out = w0->n_out; a.k_div = k_div;
    a.groups = (const PGroup *)groups; a.n_groups = n_groups; a.row_to_pair = row_to_pair;
    a.in_hi = (const __half *)in_hi; a.in_lo = (const __half *)in_lo; a.sum_hi = (const __half *)sum_hi; a.sum_lo = (const __half *)sum_lo;
    a.out_hi = (__half *)out_hi; a.out_lo = (__half *)out_lo; a.osum_hi = (__half *)osum_hi; a.osum_lo = (__half *)osum_lo;
    a.out = out; a.status = status; a.debug = g_prefill_debug ? g_prefill_debug + 32 * mode : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (mode == 0) {
        e = cudaFuncSetAttribute(prefill_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PT_SMEM);
        if (e != cudaSuccess) return (int)e;
        prefill_tc_kernel<0><<<ctas, PT_THREADS, PT_SMEM, s>>>(m0, m1, a);
    } else {
        e = cudaFuncSetAttribute(prefill_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PT_SMEM);
        if (e != cudaSuccess) return (int)e;
        prefill_tc_kernel<1><<<ctas, PT_THREADS, PT_SMEM, s>>>(m0, m1, a);
    }
    return qw4sh_note_launch("prefill_tc_kernel");
}
