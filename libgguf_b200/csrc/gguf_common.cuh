// Shared device/host helpers of the B200 GGUF row kernels: block geometry, the exact scalar
// conversions, rounding helpers and the packed IQ codebooks.
//
// Exactness contract: every float expression in this tree is evaluated as written, in fp32,
// without fused multiply-add (the translation units are compiled with --fmad=false, IEEE
// division and square root, no flush-to-zero), because the encoded bytes must equal what the
// upstream CPU REF backend produces (upstream CMakeLists.txt:76-82 builds it with plain -O3).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/libgguf.h"

#define GGUF_HD __host__ __device__ __forceinline__
#define GGUF_D __device__ __forceinline__

namespace gguf {

constexpr int QK_K = 256;  // super-block width (upstream libgguf_internal.h:62)

// Elements and bytes of one encoded block per type (upstream libgguf_internal.h:146-458).
struct BlockGeom {
    int elems;
    int bytes;
};

GGUF_HD BlockGeom block_geom(int type) {
    switch (type) {
        case GGML_TYPE_Q4_0: return {32, 18};
        case GGML_TYPE_Q4_1: return {32, 20};
        case GGML_TYPE_Q5_0: return {32, 22};
        case GGML_TYPE_Q5_1: return {32, 24};
        case GGML_TYPE_Q8_0: return {32, 34};
        case GGML_TYPE_Q1_0: return {128, 18};
        case GGML_TYPE_MXFP4: return {32, 17};
        case GGML_TYPE_NVFP4: return {64, 36};
        case GGML_TYPE_Q2_K: return {256, 84};
        case GGML_TYPE_Q3_K: return {256, 110};
        case GGML_TYPE_Q4_K: return {256, 144};
        case GGML_TYPE_Q5_K: return {256, 176};
        case GGML_TYPE_Q6_K: return {256, 210};
        case GGML_TYPE_TQ1_0: return {256, 54};
        case GGML_TYPE_TQ2_0: return {256, 66};
        case GGML_TYPE_IQ2_XXS: return {256, 66};
        case GGML_TYPE_IQ2_XS: return {256, 74};
        case GGML_TYPE_IQ2_S: return {256, 82};
        case GGML_TYPE_IQ3_XXS: return {256, 98};
        case GGML_TYPE_IQ3_S: return {256, 110};
        case GGML_TYPE_IQ1_S: return {256, 50};
        case GGML_TYPE_IQ1_M: return {256, 56};
        case GGML_TYPE_IQ4_NL: return {32, 18};
        case GGML_TYPE_IQ4_XS: return {256, 136};
        default: return {0, 0};
    }
}

// ---------------------------------------------------------------------------------------------
// bit casts
GGUF_HD float bits_to_f32(uint32_t u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    union { uint32_t u; float f; } c; c.u = u; return c.f;
#endif
}
GGUF_HD uint32_t f32_to_bits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    union { uint32_t u; float f; } c; c.f = f; return c.u;
#endif
}

// fp16 -> fp32, same integer/float steps as upstream libgguf_common.h:28-50 so that NaN payloads
// and subnormals come out with identical bits.
GGUF_HD float half_bits_to_f32(uint16_t h) {
    const uint32_t w = (uint32_t)h << 16;
    const uint32_t sign = w & 0x80000000u;
    const uint32_t two_w = w + w;
    const float normalized = bits_to_f32((two_w >> 4) + (0xE0u << 23)) * bits_to_f32(0x07800000u);  // * 2^-112
    const float denormalized = bits_to_f32((two_w >> 17) | (126u << 23)) - 0.5f;
    const uint32_t r = sign | (two_w < (1u << 27) ? f32_to_bits(denormalized) : f32_to_bits(normalized));
    return bits_to_f32(r);
}

// fp32 -> fp16 round-to-nearest-even, NaN -> sign|0x7E00 (upstream libgguf_common.h:52-78).
GGUF_HD uint16_t f32_to_half_bits(float f) {
    float base = (fabsf(f) * bits_to_f32(0x77800000u)) * bits_to_f32(0x08800000u);  // *2^112 then *2^-110
    const uint32_t w = f32_to_bits(f);
    const uint32_t shl1_w = w + w;
    const uint32_t sign = w & 0x80000000u;
    uint32_t bias = shl1_w & 0xFF000000u;
    if (bias < 0x71000000u) bias = 0x71000000u;
    base = bits_to_f32((bias >> 1) + 0x07800000u) + base;
    const uint32_t bits = f32_to_bits(base);
    const uint32_t exp_bits = (bits >> 13) & 0x00007C00u;
    const uint32_t mantissa_bits = bits & 0x00000FFFu;
    const uint32_t nonsign = exp_bits + mantissa_bits;
    return (uint16_t)((sign >> 16) | (shl1_w > 0xFF000000u ? 0x7E00u : nonsign));
}

// fp32 -> bf16 round-to-nearest-even, NaN quieted with its payload kept
// (upstream libgguf_common.h:280-296).
GGUF_HD uint16_t f32_to_bf16_bits(float s) {
    const uint32_t i = f32_to_bits(s);
    if ((i & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((i >> 16) | 64);
    return (uint16_t)((i + (0x7fffu + ((i >> 16) & 1))) >> 16);
}

// E8M0 exponent byte -> 2^(x-128), i.e. half of the E8M0 value (upstream libgguf_common.h:124-145).
GGUF_HD float e8m0_half_to_f32(uint8_t x) {
    const uint32_t bits = x < 2 ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23);
    return bits_to_f32(bits);
}

// UE4M3 byte -> half of its value (upstream libgguf_common.h:152-171).  ldexpf by a power of two
// is exact, so the value is rebuilt from exact products.
GGUF_HD float ue4m3_half_to_f32(uint8_t x) {
    if (x == 0 || x == 0x7F) return 0.0f;
    const int exp = (x >> 3) & 0xF;
    const int man = x & 0x7;
    // normal codes: (1 + man/8) * 2^(exp-7) * 0.5 written directly as float bits
    if (exp != 0) return bits_to_f32(((uint32_t)(exp + 119) << 23) | ((uint32_t)man << 20));
    float raw;
    if (exp == 0) {
        raw = (float)man * bits_to_f32((127u - 9u) << 23);
    } else {
        raw = (1.0f + (float)man / 8.0f) * bits_to_f32((uint32_t)(exp - 7 + 127) << 23);
    }
    return raw * 0.5f;
}

// fp32 -> UE4M3 with upstream's rounding (bit 19 decides, subnormals by x*512+0.5 truncation;
// upstream libgguf_common.h:173-220).
GGUF_HD uint8_t f32_to_ue4m3(float x) {
    if (!(x > 0.0f)) return 0;
    if (x > 448.0f) x = 448.0f;
    const uint32_t bits = f32_to_bits(x);
    const int fp32_exp = (int)((bits >> 23) & 0xFF) - 127;
    const int fp32_man = (bits >> 20) & 0x7;
    int ue_exp = fp32_exp + 7;
    if (ue_exp <= 0) {
        int man = (int)(x * 512.0f + 0.5f);
        if (man > 7) man = 7;
        if (man < 1) return 0;
        return (uint8_t)man;
    }
    if (ue_exp >= 15) return 0x7E;
    const int round_bit = (bits >> 19) & 1;
    int ue_man = fp32_man + round_bit;
    if (ue_man > 7) {
        ue_man = 0;
        ue_exp++;
        if (ue_exp >= 15) return 0x7E;
    }
    return (uint8_t)((ue_exp << 3) | ue_man);
}

// Round to nearest integer, ties to even, by the 1.5*2^23 trick (upstream libgguf_common.h:337-344).
GGUF_HD int nearest_int(float fval) {
    const float val = fval + 12582912.f;
    return (int)(f32_to_bits(val) & 0x007fffffu) - 0x00400000;
}

GGUF_HD int imin(int a, int b) { return a < b ? a : b; }
GGUF_HD int imax(int a, int b) { return a > b ? a : b; }

// (int8_t)(float) as x86 does it: truncate to int32 (out of range / NaN -> INT_MIN), keep the low byte.
GGUF_HD int cast_f32_to_i8_x86(float v) {
    int i;
    if (v >= 2147483648.0f || v < -2147483648.0f || v != v) i = (int)0x80000000;
    else i = (int)v;
    return (int)(int8_t)(i & 0xFF);
}

// Kernel launch geometry helper.
inline unsigned blocks_for(int64_t n, int per_block) { return (unsigned)((n + per_block - 1) / per_block); }

// ---------------------------------------------------------------------------------------------
// Codebooks.  kvalues: upstream libgguf_tables.cpp:615-628.
#ifdef __CUDACC__
#define GGUF_TABLE __device__ const
#else
#define GGUF_TABLE static const
#endif

}  // namespace gguf
