// Device-side GGUF block decoders over the RESIDENT weight image.
//
// Decoded values are bit-identical to picoforge's CPU decoder (src/qwen4_packed.c:54-122):
// every product and difference below is an explicitly rounded binary32 operation
// (__fmul_rn / __fsub_rn are never contracted into FMAs).
//
// Resident layout.  A tensor is [expert][row][packed K] on the host.  On the device each
// expert matrix keeps its byte size and its offset (expert * expert_bytes), but two
// formats are regrouped INSIDE the matrix so that every field is naturally aligned:
//
//   Q4_K     unchanged: block b of row n at (n * nb + b) * 144; 144 = 9 * 16 bytes.
//   Q2_K     [rows*nb][64 B codes] | [rows*nb][16 B scale/min bytes] | [rows*nb][d, dmin f16]
//   IQ2_XXS  [rows][nb*8 groups x 8 B] | [rows*nb][d f16]; inside a row, 8-byte group c is
//            stored at position c ^ ((row & 3) << 2) (rows of two or more blocks), so that the
//            four rows a half-warp reads together fall in different shared-memory banks when
//            whole row tiles are copied to shared memory unchanged
//   others   unchanged (F32, F16, BF16, Q8_0, MXFP4).
//
// nb = k_storage / 256.  The regrouping is a permutation of bytes done once at upload.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "iq2xxs_codebook.h"

namespace qw4 {

enum : uint32_t { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_Q2_K = 10, T_Q4_K = 12, T_IQ2_XXS = 16, T_BF16 = 30, T_MXFP4 = 39 };

// One resident tensor.  Plain data: passed to kernels by value.
struct DevTensor {
    const uint8_t *data;
    uint32_t type;
    uint32_t k_storage, k_logical, n_out, n_experts;
    uint32_t row_bytes;
    uint64_t expert_bytes;
};

// Statically initialised per translation unit: no runtime copy is needed.
static __device__ __constant__ uint16_t c_iq2_levels[256] = { QW4_IQ2XXS_LEVEL_LIST };

__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    return __half2float(__ushort_as_half(h));          // exact, subnormals included
}
__device__ __forceinline__ uint32_t load_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
__device__ __forceinline__ uint32_t load_u32(const uint8_t *p) { return *reinterpret_cast<const uint32_t *>(p); }

__device__ __forceinline__ uint32_t iq2_magnitude(uint32_t level) { return 8u + 17u * level + (level >> 1); }

// Position swizzle of IQ2_XXS groups inside a row of the resident image.
__host__ __device__ __forceinline__ uint32_t iq2_swizzle(uint32_t row, uint32_t nb) { return nb >= 2 ? (row & 3u) << 2 : 0u; }

// 8th sign of an IQ2_XXS vector: parity of the seven stored ones.
__device__ __forceinline__ uint32_t iq2_signs8(uint32_t seven) { return seven | ((__popc(seven) & 1u) << 7); }

// Q4_K scale and min of sub-block g from the 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(const uint8_t *sc, uint32_t g, uint32_t &scale, uint32_t &minimum) {
    if (g < 4) { scale = sc[g] & 63u; minimum = sc[g + 4] & 63u; }
    else {
        scale = (sc[g + 4] & 15u) | ((sc[g - 4] & 192u) >> 2);
        minimum = (uint32_t)(sc[g + 4] >> 4) | ((sc[g] & 192u) >> 2);
    }
}

// Value of weight (expert, row, column) of a resident tensor, exact.  Slow path used by
// the decode probe, the generic any-format kernels and as the definition the fast kernels
// are tested against.
__device__ inline float decode_value(const DevTensor &t, uint32_t expert, uint32_t row, uint32_t column) {
    const uint8_t *mat = t.data + (uint64_t)expert * t.expert_bytes;
    const uint32_t nb = t.k_storage >> 8;
    switch (t.type) {
    case T_F32: return __uint_as_float(load_u32(mat + (uint64_t)row * t.row_bytes + 4u * column));
    case T_F16: return half_bits_to_float((uint16_t)load_u16(mat + (uint64_t)row * t.row_bytes + 2u * column));
    case T_BF16: return __uint_as_float(load_u16(mat + (uint64_t)row * t.row_bytes + 2u * column) << 16);
    case T_Q8_0: {
        const uint8_t *b = mat + (uint64_t)row * t.row_bytes + (column >> 5) * 34u;
        const int code = (int)(int8_t)b[2 + (column & 31u)];
        return __fmul_rn(half_bits_to_float((uint16_t)load_u16(b)), (float)code);
    }
    case T_MXFP4: {
        const uint8_t *b = mat + (uint64_t)row * t.row_bytes + (column >> 5) * 17u;
        const uint32_t lane = column & 31u, code = (b[1 + (lane & 15u)] >> ((lane >> 4) * 4)) & 15u;
        const float table[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
        const float value = (code & 8u) ? -table[code & 7u] : table[code & 7u];
        const float scale = __uint_as_float(b[0] ? (uint32_t)b[0] << 23 : 0x00400000u);
        return __fmul_rn(value, scale);
    }
    case T_Q4_K: {
        const uint8_t *b = mat + ((uint64_t)row * nb + (column >> 8)) * 144u;
        const uint32_t lane = column & 255u, g = lane >> 5;
        uint32_t scale, minimum;
        q4k_scale_min(b + 4, g, scale, minimum);
        const uint32_t code = (b[16 + (g >> 1) * 32 + (lane & 31u)] >> ((g & 1u) * 4)) & 15u;
        const float d = half_bits_to_float((uint16_t)load_u16(b)), dmin = half_bits_to_float((uint16_t)load_u16(b + 2));
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)scale), (float)code), __fmul_rn(dmin, (float)minimum));
    }
    case T_Q2_K: {
        const uint64_t blocks = (uint64_t)t.n_out * nb, block = (uint64_t)row * nb + (column >> 8);
        const uint8_t *codes = mat + block * 64u, *scales = mat + blocks * 64u + block * 16u;
        const uint8_t *dd = mat + blocks * 80u + block * 4u;
        const uint32_t lane = column & 255u, s = scales[lane >> 4];
        const uint32_t code = (codes[(lane >> 7) * 32 + (lane & 31u)] >> (2 * ((lane & 127u) >> 5))) & 3u;
        const float d = half_bits_to_float((uint16_t)load_u16(dd)), dmin = half_bits_to_float((uint16_t)load_u16(dd + 2));
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)(s & 15u)), (float)code), __fmul_rn(dmin, (float)(s >> 4)));
    }
    case T_IQ2_XXS: {
        const uint64_t blocks = (uint64_t)t.n_out * nb, block = (uint64_t)row * nb + (column >> 8);
        const uint32_t lane = column & 255u, slot = (lane & 31u) >> 3;
        const uint8_t *group = mat + ((uint64_t)row * nb * 8u + ((((column >> 8) * 8u) + (lane >> 5)) ^ iq2_swizzle(row, nb))) * 8u;
        const uint32_t bits = load_u32(group + 4);
        const uint32_t signs = iq2_signs8((bits >> (7 * slot)) & 127u);
        const uint32_t level = (c_iq2_levels[group[slot]] >> (2 * (lane & 7u))) & 3u;
        const float d = half_bits_to_float((uint16_t)load_u16(mat + blocks * 64u + block * 2u));
        const float scale = __fmul_rn(__fmul_rn(d, (float)(2u * (bits >> 28) + 1u)), 0.125f);
        const float value = __fmul_rn(scale, (float)iq2_magnitude(level));
        return (signs >> (lane & 7u)) & 1u ? -value : value;
    }
    default: return __uint_as_float(0x7fc00000u);
    }
}

// The hyper-connection add that follows the layer (picoforge src/qwen4_base.c:160-176, fused into the down
// epilogue by the reference's GPU path, src/qwen4_moe_internal.h:55-58): for each of the `streams` residual
// streams, residual[t, h, c] += inject[t, h] * y[t, c], the product and the sum rounded separately.  Called by
// whichever thread writes y[t, c]; returns false when a result is not finite.
struct HcAdd {
    float *residual;                    // [tokens, streams, hidden]; nullptr: no add
    const float *inject;                // [tokens, streams]
    uint32_t streams;
};
__device__ __forceinline__ bool hc_add(const HcAdd &hc, uint32_t t, uint32_t c, uint32_t hidden, float y) {
    if (!hc.residual) return true;
    bool ok = true;
    for (uint32_t h = 0; h < hc.streams; h++) {
        float *at = hc.residual + ((uint64_t)t * hc.streams + h) * hidden + c;
        const float r = __fadd_rn(*at, __fmul_rn(hc.inject[(uint64_t)t * hc.streams + h], y));
        ok &= (__float_as_uint(r) & 0x7f800000u) != 0x7f800000u;
        *at = r;
    }
    return ok;
}

}  // namespace qw4
