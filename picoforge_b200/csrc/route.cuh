// Device functions shared by the routing kernels: libm-exact expf / sigmoid and the
// warp-per-token softmax + top-k (picoforge src/qwen4_moe.c:209-247).
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "cuda_shim.h"

namespace qw4 {

// ------------------------------------------------------------------------------------
// expf with glibc's bits.
//
// The reference computes softmax and sigmoid with libm expf (picoforge src/qwen4_moe.c:228,
// src/qwen4_cpu_internal.h:103-106).  glibc's expf is the table-driven double-precision
// algorithm published in ARM's optimized routines (N = 32 table, cubic polynomial); on x86-64
// machines with FMA its products and sums are fused.  Restating it with explicit fma() gives
// the same binary32 result as glibc 2.39 for every input <= 0 (1 120 927 745 values checked
// on the CPU), which is the whole domain used here: z - max <= 0 and -|x|.
// ------------------------------------------------------------------------------------
// In global (not constant) memory: lanes index it with different k, which the constant cache
// would serialise; the 256 bytes stay in L1.
static __device__ const unsigned long long c_exp2_table[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
};
// `table` may point at a copy of c_exp2_table in shared memory.
__device__ __forceinline__ float expf_libm_table(float x, const unsigned long long *table) {          // x <= 0 (or +0)
    if (x < -0x1.9fe368p6f) return 0.0f;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32, c1 = 0x1.ebfce50fac4f3p-3 / 32 / 32, c2 = 0x1.62e42ff0c52d6p-1 / 32;
    const double xd = (double)x;
    double kd = fma(inv_ln2_n, xd, shift);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, shift);
    const double r = fma(inv_ln2_n, xd, -kd);
    unsigned long long t = table[ki & 31u];
    t += ki << 47;
    const double s = __longlong_as_double((long long)t);
    const double z = fma(c0, r, c1), r2 = __dmul_rn(r, r);
    double y = fma(c2, r, 1.0);
    y = fma(z, r2, y);
    return __double2float_rn(__dmul_rn(y, s));
}
__device__ __forceinline__ float expf_libm(float x) { return expf_libm_table(x, c_exp2_table); }
__device__ __forceinline__ float sigmoid_libm(float x) {      // src/qwen4_cpu_internal.h:103-106
    if (x >= 0.0f) return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_libm(-x)));
    const float z = expf_libm(x);
    return __fdiv_rn(z, __fadd_rn(1.0f, z));
}
__device__ __forceinline__ bool finite_f32(float v) { return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u; }

// One token per warp, for experts <= 32 * PL, with the token's probabilities in registers: lane L holds
// experts L, L + 32, ...  The exp-sum still runs in expert order (e = 0, 1, 2, ...): every lane
// fetches the values one by one with shuffles and adds them in that order.  Returns false (and
// records the row) when a logit is not finite; ids and weights are then left untouched.
template <int PL>
__device__ __forceinline__ bool route_token_regs(uint32_t experts, uint32_t k, int norm, const float *__restrict__ z, uint32_t t,
                                                 float *__restrict__ probs, uint32_t *__restrict__ ids, float *__restrict__ weights,
                                                 uint32_t *status, uint32_t lane) {
    float p[PL];
    bool bad = false;
    float maximum = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < PL; i++) {
        const uint32_t e = lane + 32 * i;
        p[i] = e < experts ? z[e] : -CUDART_INF_F;
        if (e < experts) { bad |= !finite_f32(p[i]); maximum = fmaxf(maximum, p[i]); }
    }
    bad = __any_sync(0xffffffffu, bad);
    if (bad) {
        if (lane == 0) { atomicOr(status, QW4SH_ERR_NONFINITE); atomicMin(status + 1, t); }
        return false;
    }
    for (int o = 16; o; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
#pragma unroll
    for (int i = 0; i < PL; i++) p[i] = lane + 32 * i < experts ? expf_libm(__fsub_rn(p[i], maximum)) : 0.0f;
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < PL; i++) {
        if (32u * i >= experts) break;
        const uint32_t n = min(32u, experts - 32u * i);
        if (n == 32) {
#pragma unroll
            for (int l = 0; l < 32; l++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, p[i], l));
        } else {
            for (uint32_t l = 0; l < n; l++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, p[i], l));
        }
    }
#pragma unroll
    for (int i = 0; i < PL; i++) {
        const uint32_t e = lane + 32 * i;
        if (e < experts) { p[i] = __fdiv_rn(p[i], sum); if (probs) probs[(uint64_t)t * experts + e] = p[i]; }
        else p[i] = -1.0f;
    }
    float selected = 0.0f, mine = 0.0f;                        // lane s keeps the weight of slot s
    for (uint32_t slot = 0; slot < k; slot++) {
        float best = -1.0f;
        uint32_t best_e = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < PL; i++) if (p[i] > best) { best = p[i]; best_e = lane + 32 * i; }
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (lane == 0) ids[(uint64_t)t * k + slot] = best_e;
        if ((slot & 31u) == lane) mine = best;                 // k <= 32 on this path
        if ((best_e & 31u) == lane) {
#pragma unroll
            for (int i = 0; i < PL; i++) if ((uint32_t)i == (best_e >> 5)) p[i] = -1.0f;
        }
        selected = __fadd_rn(selected, best);
    }
    if (lane < k) weights[(uint64_t)t * k + lane] = norm ? __fdiv_rn(mine, selected) : mine;
    return true;
}


}  // namespace qw4
