// Row decoders: packed GGUF blocks -> fp32 / fp16 / bf16.
//
// One kernel template serves every type.  A CTA owns a tile of consecutive blocks:
//   1. the tile's bytes are staged into shared memory with 16-byte loads from the 16-byte
//      aligned span that covers it (block sizes such as 34, 110 or 210 bytes make per-block
//      vector loads impossible; a span of blocks does not care),
//   2. every thread decodes runs of 8 consecutive output elements from shared memory, so a warp
//      writes 32 x 16 B (fp16/bf16) or 2 x 32 x 16 B (fp32) of contiguous output per step.
// The arithmetic of each decoder follows the upstream scalar decoder expression by expression
// (upstream csrc/dequant/dequant.cpp); products are formed in the same order because fp32
// output must be bit-identical.  fp16/bf16 output is the round-to-nearest-even conversion of
// that fp32 value.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "gguf_common.cuh"
#include "gguf_tables.cuh"
#include "kernels.h"

namespace gguf {
namespace {

GGUF_D uint16_t ld16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
GGUF_D uint32_t ld32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

// 6-bit scale / min pair j of a Q4_K / Q5_K block (upstream libgguf_common.h:672-684).
GGUF_D void scale_min_k4(int j, const uint8_t *q, int &sc, int &m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

template <int TYPE>
struct Decoder;

// upstream dequant.cpp:120-134
template <>
struct Decoder<GGML_TYPE_Q8_0> {
    static constexpr int ELEMS = 32, BYTES = 34;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)(int8_t)b[2 + e0 + i] * d;
    }
};

// upstream dequant.cpp:21-35
template <>
struct Decoder<GGML_TYPE_Q4_0> {
    static constexpr int ELEMS = 32, BYTES = 18;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int sh = e0 >= 16 ? 4 : 0;
        const uint8_t *q = b + 2 + (e0 & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)(((q[i] >> sh) & 0xF) - 8) * d;
    }
};

// upstream dequant.cpp:37-52
template <>
struct Decoder<GGML_TYPE_Q4_1> {
    static constexpr int ELEMS = 32, BYTES = 20;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const float m = half_bits_to_f32(ld16(b + 2));
        const int sh = e0 >= 16 ? 4 : 0;
        const uint8_t *q = b + 4 + (e0 & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)((q[i] >> sh) & 0xF) * d + m;
    }
};

// upstream dequant.cpp:54-76
template <>
struct Decoder<GGML_TYPE_Q5_0> {
    static constexpr int ELEMS = 32, BYTES = 22;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const uint32_t qh = ld32(b + 2);
        const int sh = e0 >= 16 ? 4 : 0;
        const uint8_t *q = b + 6 + (e0 & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int hi = (int)((qh >> (e0 + i)) & 1) << 4;
            v[i] = (float)((((q[i] >> sh) & 0xF) | hi) - 16) * d;
        }
    }
};

// upstream dequant.cpp:78-101
template <>
struct Decoder<GGML_TYPE_Q5_1> {
    static constexpr int ELEMS = 32, BYTES = 24;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const float m = half_bits_to_f32(ld16(b + 2));
        const uint32_t qh = ld32(b + 4);
        const int sh = e0 >= 16 ? 4 : 0;
        const uint8_t *q = b + 8 + (e0 & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int hi = (int)((qh >> (e0 + i)) & 1) << 4;
            v[i] = (float)(((q[i] >> sh) & 0xF) | hi) * d + m;
        }
    }
};

// upstream dequant.cpp:6-19
template <>
struct Decoder<GGML_TYPE_Q1_0> {
    static constexpr int ELEMS = 128, BYTES = 18;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const float neg_d = -d;
        const uint32_t bits = b[2 + (e0 >> 3)];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = ((bits >> i) & 1) ? d : neg_d;
    }
};

// upstream dequant.cpp:136-154
template <>
struct Decoder<GGML_TYPE_MXFP4> {
    static constexpr int ELEMS = 32, BYTES = 17;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = e8m0_half_to_f32(b[0]);
        const int sh = e0 >= 16 ? 4 : 0;
        const uint8_t *q = b + 1 + (e0 & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)k_fp4_values[(q[i] >> sh) & 0xF] * d;
    }
};

// upstream dequant.cpp:156-179
template <>
struct Decoder<GGML_TYPE_NVFP4> {
    static constexpr int ELEMS = 64, BYTES = 36;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const int s = e0 >> 4;
        const float d = ue4m3_half_to_f32(b[s]);
        const int sh = (e0 & 8) ? 4 : 0;
        const uint8_t *q = b + 4 + s * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)k_fp4_values[(q[i] >> sh) & 0xF] * d;
    }
};

// upstream dequant.cpp:181-211.  Element e: half n = e/128, 2-bit plane j = (e%128)/32,
// 16-wide group (e%32)/16; scale byte index 8n + 2j + group.
template <>
struct Decoder<GGML_TYPE_Q2_K> {
    static constexpr int ELEMS = 256, BYTES = 84;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b + 80));
        const float dmin = half_bits_to_f32(ld16(b + 82));
        const int n = e0 >> 7, j = (e0 >> 5) & 3, r = e0 & 31;
        const int sc = b[8 * n + 2 * j + (r >> 4)];
        const float dl = d * (float)(sc & 0xF);
        const float ml = dmin * (float)(sc >> 4);
        const uint8_t *q = b + 16 + 32 * n + r;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * (float)((q[i] >> (2 * j)) & 3) - ml;
    }
};

// upstream dequant.cpp:213-261
template <>
struct Decoder<GGML_TYPE_Q3_K> {
    static constexpr int ELEMS = 256, BYTES = 110;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d_all = half_bits_to_f32(ld16(b + 108));
        const int n = e0 >> 7, j = (e0 >> 5) & 3, r = e0 & 31;
        const int is = 8 * n + 2 * j + (r >> 4);
        // 6-bit scale `is`: low nibble from scales[is%8] (high nibble for is>=8), top 2 bits from scales[8 + is%4].
        const uint8_t *s = b + 96;
        const int lo = is < 8 ? (s[is] & 0xF) : (s[is - 8] >> 4);
        const int hi = (s[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
        const float dl = d_all * (float)((int)(int8_t)(lo | (hi << 4)) - 32);
        const uint8_t *q = b + 32 + 32 * n + r;
        const uint8_t *hm = b + r;
        const int mbit = 1 << (4 * n + j);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int ql = (q[i] >> (2 * j)) & 3;
            v[i] = dl * (float)(ql - ((hm[i] & mbit) ? 0 : 4));
        }
    }
};

// upstream dequant.cpp:263-285
template <>
struct Decoder<GGML_TYPE_Q4_K> {
    static constexpr int ELEMS = 256, BYTES = 144;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const float dmin = half_bits_to_f32(ld16(b + 2));
        const int j64 = e0 >> 6, hi = (e0 >> 5) & 1, l0 = e0 & 31;
        int sc, m;
        scale_min_k4(2 * j64 + hi, b + 4, sc, m);
        const float d1 = d * (float)sc;
        const float m1 = dmin * (float)m;
        const uint8_t *q = b + 16 + 32 * j64 + l0;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d1 * (float)((q[i] >> (4 * hi)) & 0xF) - m1;
    }
};

// upstream dequant.cpp:287-312
template <>
struct Decoder<GGML_TYPE_Q5_K> {
    static constexpr int ELEMS = 256, BYTES = 176;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const float dmin = half_bits_to_f32(ld16(b + 2));
        const int j64 = e0 >> 6, hi = (e0 >> 5) & 1, l0 = e0 & 31;
        int sc, m;
        scale_min_k4(2 * j64 + hi, b + 4, sc, m);
        const float d1 = d * (float)sc;
        const float m1 = dmin * (float)m;
        const uint8_t *qh = b + 16 + l0;
        const uint8_t *q = b + 48 + 32 * j64 + l0;
        const int hbit = 1 << (2 * j64 + hi);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d1 * (float)(((q[i] >> (4 * hi)) & 0xF) + ((qh[i] & hbit) ? 16 : 0)) - m1;
    }
};

// upstream dequant.cpp:314-343
template <>
struct Decoder<GGML_TYPE_Q6_K> {
    static constexpr int ELEMS = 256, BYTES = 210;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b + 208));
        const int n = e0 >> 7, quarter = (e0 >> 5) & 3, l0 = e0 & 31;
        const int sc = (int8_t)b[192 + 8 * n + (l0 >> 4) + 2 * quarter];
        const float ds = d * (float)sc;
        const uint8_t *ql = b + 64 * n + 32 * (quarter & 1) + l0;
        const uint8_t *qh = b + 128 + 32 * n + l0;
        const int lsh = (quarter & 2) ? 4 : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int q = (int)(int8_t)(((ql[i] >> lsh) & 0xF) | (((qh[i] >> (2 * quarter)) & 3) << 4)) - 32;
            v[i] = ds * (float)q;
        }
    }
};

// upstream dequant.cpp:345-383.  Layout: 32 bytes x 5 trits, 16 bytes x 5 trits, 4 bytes x 4 trits.
template <>
struct Decoder<GGML_TYPE_TQ1_0> {
    static constexpr int ELEMS = 256, BYTES = 54;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b + 52));
        const int pow3[5] = {1, 3, 9, 27, 81};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = e0 + i;
            int byte, n;
            if (e < 160) {
                n = e >> 5;
                byte = b[e & 31];
            } else if (e < 240) {
                n = (e - 160) >> 4;
                byte = b[32 + ((e - 160) & 15)];
            } else {
                n = (e - 240) >> 2;
                byte = b[48 + ((e - 240) & 3)];
            }
            const int q = (byte * pow3[n]) & 0xFF;
            const int xi = (q * 3) >> 8;
            v[i] = (float)(xi - 1) * d;
        }
    }
};

// upstream dequant.cpp:385-401
template <>
struct Decoder<GGML_TYPE_TQ2_0> {
    static constexpr int ELEMS = 256, BYTES = 66;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b + 64));
        const int j = e0 >> 7, l = (e0 >> 5) & 3, m0 = e0 & 31;
        const uint8_t *q = b + 32 * j + m0;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)(((q[i] >> (2 * l)) & 3) - 1) * d;
    }
};

// Eight values of one IQ2 grid point with its sign byte applied.
GGUF_D void iq2_emit(uint32_t code, uint32_t signs, float db, float *v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float g = db * (float)iq2_grid_byte((code >> (2 * i)) & 3);
        v[i] = (signs >> i) & 1 ? -g : g;
    }
}

// upstream dequant.cpp:403-427
template <>
struct Decoder<GGML_TYPE_IQ2_XXS> {
    static constexpr int ELEMS = 256, BYTES = 66;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int ib32 = e0 >> 5, l = (e0 >> 3) & 3;
        const uint8_t *q = b + 2 + 8 * ib32;
        const uint32_t aux1 = ld32(q + 4);
        const float db = d * (0.5f + (float)(aux1 >> 28)) * 0.25f;
        iq2_emit(k_codebook_IQ2XXS[q[l]], iq_signs_from_index((aux1 >> (7 * l)) & 127), db, v);
    }
};

// upstream dequant.cpp:429-452
template <>
struct Decoder<GGML_TYPE_IQ2_XS> {
    static constexpr int ELEMS = 256, BYTES = 74;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int g = e0 >> 3, ib32 = g >> 2, l = g & 3;
        const uint32_t q = ld16(b + 2 + 2 * g);
        const int sc = b[66 + ib32];
        const float db = d * (0.5f + (float)((l < 2) ? (sc & 0xF) : (sc >> 4))) * 0.25f;
        iq2_emit(k_codebook_IQ2XS[q & 511], iq_signs_from_index(q >> 9), db, v);
    }
};

// upstream dequant.cpp:454-482
template <>
struct Decoder<GGML_TYPE_IQ2_S> {
    static constexpr int ELEMS = 256, BYTES = 82;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int g = e0 >> 3, ib32 = g >> 2, l = g & 3;
        const int sc = b[74 + ib32];
        const float db = d * (0.5f + (float)((l < 2) ? (sc & 0xF) : (sc >> 4))) * 0.25f;
        const uint32_t idx = b[2 + g] | (((uint32_t)b[66 + ib32] << (8 - 2 * l)) & 0x300);
        iq2_emit(k_codebook_IQ2S[idx], b[2 + 32 + g], db, v);
    }
};

// upstream dequant.cpp:484-512
template <>
struct Decoder<GGML_TYPE_IQ3_XXS> {
    static constexpr int ELEMS = 256, BYTES = 98;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int g = e0 >> 3, ib32 = g >> 2, l = g & 3;
        const uint32_t aux = ld32(b + 2 + 64 + 4 * ib32);
        const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
        const uint32_t signs = iq_signs_from_index((aux >> (7 * l)) & 127);
        const uint32_t c1 = k_codebook_IQ3XXS[b[2 + 2 * g]];
        const uint32_t c2 = k_codebook_IQ3XXS[b[2 + 2 * g + 1]];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float g1 = db * (float)iq3xxs_grid_byte((c1 >> (3 * i)) & 7);
            const float g2 = db * (float)iq3xxs_grid_byte((c2 >> (3 * i)) & 7);
            v[i] = (signs >> i) & 1 ? -g1 : g1;
            v[i + 4] = (signs >> (i + 4)) & 1 ? -g2 : g2;
        }
    }
};

// upstream dequant.cpp:630-669
template <>
struct Decoder<GGML_TYPE_IQ3_S> {
    static constexpr int ELEMS = 256, BYTES = 110;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int g = e0 >> 3, ib32 = g >> 2, l = g & 3;
        const int sc = b[106 + (ib32 >> 1)];
        const float db = d * (float)(1 + 2 * ((ib32 & 1) ? (sc >> 4) : (sc & 0xF)));
        const uint32_t qh = b[66 + ib32];
        const uint32_t i1 = b[2 + 2 * g] | ((qh << (8 - 2 * l)) & 256);
        const uint32_t i2 = b[2 + 2 * g + 1] | ((qh << (7 - 2 * l)) & 256);
        const uint32_t signs = b[74 + g];
        const uint32_t c1 = k_codebook_IQ3S[i1];
        const uint32_t c2 = k_codebook_IQ3S[i2];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float g1 = db * (float)iq3s_grid_byte((c1 >> (3 * i)) & 7);
            const float g2 = db * (float)iq3s_grid_byte((c2 >> (3 * i)) & 7);
            v[i] = (signs >> i) & 1 ? -g1 : g1;
            v[i + 4] = (signs >> (i + 4)) & 1 ? -g2 : g2;
        }
    }
};

// upstream dequant.cpp:514-538
template <>
struct Decoder<GGML_TYPE_IQ1_S> {
    static constexpr int ELEMS = 256, BYTES = 50;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int g = e0 >> 3, ib = g >> 2, l = g & 3;
        const uint32_t qh = ld16(b + 34 + 2 * ib);
        const float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
        const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
        const uint32_t code = k_codebook_IQ1S[b[2 + g] | (((qh >> (3 * l)) & 7) << 8)];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * ((float)iq1_grid_value((code >> (2 * i)) & 3) + delta);
    }
};

// upstream dequant.cpp:540-587
template <>
struct Decoder<GGML_TYPE_IQ1_M> {
    static constexpr int ELEMS = 256, BYTES = 56;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const uint32_t s0 = ld16(b + 48), s1 = ld16(b + 50), s2 = ld16(b + 52), s3 = ld16(b + 54);
        const uint16_t dbits = (uint16_t)((s0 >> 12) | ((s1 >> 8) & 0x00f0) | ((s2 >> 4) & 0x0f00) | (s3 & 0xf000));
        const float d = half_bits_to_f32(dbits);
        const int g = e0 >> 3, ib = g >> 2, l = g & 3;
        const uint32_t sc = ld16(b + 48 + 2 * (ib >> 1));
        const float dl = d * (float)(2 * ((sc >> (6 * (ib & 1) + (l >= 2 ? 3 : 0))) & 7) + 1);
        const uint32_t qh = b[32 + 2 * ib + (l >> 1)];
        const uint32_t idx = b[g] | ((qh << ((l & 1) ? 4 : 8)) & 0x700);
        const float delta = (qh & ((l & 1) ? 0x80 : 0x08)) ? -0.125f : 0.125f;
        const uint32_t code = k_codebook_IQ1S[idx];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * ((float)iq1_grid_value((code >> (2 * i)) & 3) + delta);
    }
};

// upstream dequant.cpp:589-603
template <>
struct Decoder<GGML_TYPE_IQ4_NL> {
    static constexpr int ELEMS = 32, BYTES = 18;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int sh = e0 >= 16 ? 4 : 0;
        const uint8_t *q = b + 2 + (e0 & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d * (float)k_iq4nl_values[(q[i] >> sh) & 0xF];
    }
};

// upstream dequant.cpp:605-628
template <>
struct Decoder<GGML_TYPE_IQ4_XS> {
    static constexpr int ELEMS = 256, BYTES = 136;
    static GGUF_D void run(const uint8_t *b, int e0, float *v) {
        const float d = half_bits_to_f32(ld16(b));
        const int ib = e0 >> 5, r = e0 & 31;
        const uint32_t scales_h = ld16(b + 2);
        const int ls = ((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (((scales_h >> (2 * ib)) & 3) << 4);
        const float dl = d * (float)(ls - 32);
        const int sh = r >= 16 ? 4 : 0;
        const uint8_t *q = b + 8 + 16 * ib + (r & 15);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * (float)k_iq4nl_values[(q[i] >> sh) & 0xF];
    }
};

// bf16 storage "decoder": widen by shifting into the high half (upstream libgguf_common.h:262-271).
template <>
struct Decoder<GGML_TYPE_BF16> {
    static constexpr int ELEMS = 8, BYTES = 16;
    static GGUF_D void run(const uint8_t *b, int, float *v) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bits_to_f32((uint32_t)ld16(b + 2 * i) << 16);
    }
};

// ---------------------------------------------------------------------------------------------
// Fast decoders for the types the bandwidth targets are quoted on.  Same arithmetic as the
// generic decoders above, restructured to spend few instructions per element (the generic kernel
// is limited by instruction issue, not by memory):
//   * constants shared by a group of 16 or 32 elements (d*scale, dmin*min) are computed once per
//     group by a first pass over the staged tile and parked in shared memory;
//   * a thread decodes 16 consecutive elements and writes them with one 256-bit store;
//   * quants are pulled out of 32-bit words four at a time and turned into floats by dropping
//     each byte into the mantissa of 2^23 (PRMT) and subtracting 2^23 plus the format's offset,
//     which is exact and avoids the integer-to-float conversion pipe;
//   * the subtract / multiply / subtract run as packed two-wide fp32 instructions (add.f32x2,
//     mul.f32x2 on sm_100), each lane rounded exactly like the scalar instruction.
// They require the encoded data to start on a 16-byte boundary and the output on a 32-byte
// boundary; otherwise the generic kernel is used.
constexpr float kTwo23 = 8388608.f;

// float(byte k of w) + 2^23
GGUF_D float magic_byte(uint32_t w, int k) { return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (uint32_t)k)); }

// 16 bytes from a shared-memory address of any alignment, via aligned 32-bit loads.
GGUF_D uint4 lds16_any(const uint8_t *p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    const uint32_t sh = (a & 3u) * 8u;
    const uint32_t *w = reinterpret_cast<const uint32_t *>(p - (a & 3u));
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
    return make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh),
                      __funnelshift_r(w3, w4, sh));
}
GGUF_D uint4 lds16_a4(const uint8_t *p) { const uint32_t *w = reinterpret_cast<const uint32_t *>(p); return make_uint4(w[0], w[1], w[2], w[3]); }
GGUF_D uint4 lds16_a16(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }
GGUF_D uint32_t lds_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
// fp16 bits -> fp32 by the hardware conversion (exact for every finite value and infinity)
GGUF_D float half_hw(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// Four quants in the bytes of w -> v[0..3] = scale * (byte - offset) [- minus], packed two-wide.
// neg_bias = -(2^23 + offset).  The assembler contracts a packed multiply that feeds a packed add into one
// fused instruction even with explicit rounding modes; that is harmless here because the product
// scale * level is exact for every type that has a second constant (an 11-bit fp16 scale times a
// sub-scale of at most 6 bits times a level of at most 5 bits), so rounding once or twice is the same.
template <bool HAS_MIN>
GGUF_D void affine4(uint32_t w, float neg_bias, float2 c, float *v) {
    const float2 nb = make_float2(neg_bias, neg_bias), sc = make_float2(c.x, c.x), nm = make_float2(-c.y, -c.y);
    float2 a = make_float2(magic_byte(w, 0), magic_byte(w, 1));
    float2 b = make_float2(magic_byte(w, 2), magic_byte(w, 3));
    a = __fmul2_rn(sc, __fadd2_rn(a, nb));
    b = __fmul2_rn(sc, __fadd2_rn(b, nb));
    if (HAS_MIN) { a = __fadd2_rn(a, nm); b = __fadd2_rn(b, nm); }
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <bool HAS_MIN>
GGUF_D void affine16(uint4 q, float neg_bias, float2 c, float *v) {
    affine4<HAS_MIN>(q.x, neg_bias, c, v);
    affine4<HAS_MIN>(q.y, neg_bias, c, v + 4);
    affine4<HAS_MIN>(q.z, neg_bias, c, v + 8);
    affine4<HAS_MIN>(q.w, neg_bias, c, v + 12);
}
GGUF_D uint4 shr_and(uint4 q, int sh, uint32_t mask) {
    return make_uint4((q.x >> sh) & mask, (q.y >> sh) & mask, (q.z >> sh) & mask, (q.w >> sh) & mask);
}
GGUF_D uint4 or_shl(uint4 q, uint4 h, int sh) { return make_uint4(q.x | (h.x << sh), q.y | (h.y << sh), q.z | (h.z << sh), q.w | (h.w << sh)); }

// scale and min code j of the 12 packed bytes of a Q4_K / Q5_K block, from its three words
GGUF_D void scale_min_words(int j, uint32_t s0, uint32_t s1, uint32_t s2, int &sc, int &m) {
    if (j < 4) {
        sc = (s0 >> (8 * j)) & 63;
        m = (s1 >> (8 * j)) & 63;
    } else {
        const int k = 8 * (j - 4);
        sc = ((s2 >> k) & 0xF) | (((s0 >> (k + 6)) & 3) << 4);
        m = ((s2 >> (k + 4)) & 0xF) | (((s1 >> (k + 6)) & 3) << 4);
    }
}

template <int TYPE>
struct Fast { static constexpr bool kEnabled = false; };

// Elements one run() call decodes: 16, or 32 for the types whose bytes hold elements j and j + 16
// (one 16-byte load then feeds both halves).
template <class D, class = void>
struct CallElems { static constexpr int value = 16; };
template <class D>
struct CallElems<D, decltype((void)D::CALL)> { static constexpr int value = D::CALL; };

// Each Fast<T>: ELEMS/BYTES of a block, GROUP = elements sharing one constant pair,
// prep(block, group index in block) and run(block, e0 (multiple of 16), constants, v[16]).
template <>
struct Fast<GGML_TYPE_Q8_0> {
    static constexpr bool kEnabled = true;
    static constexpr int TILES = 1;
    static constexpr int ELEMS = 32, BYTES = 34, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), 0.f); }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        uint4 q = lds16_any(b + 2 + e0);
        q.x ^= 0x80808080u; q.y ^= 0x80808080u; q.z ^= 0x80808080u; q.w ^= 0x80808080u;
        affine16<false>(q, -(kTwo23 + 128.f), c, v);
    }
};

template <>
struct Fast<GGML_TYPE_Q4_K> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 144, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int g) {
        const uint4 head = lds16_a16(b);  // d, dmin, 12 scale bytes
        int sc, m;
        scale_min_words(g, head.y, head.z, head.w, sc, m);
        return make_float2(half_hw(head.x & 0xFFFFu) * (float)sc, half_hw(head.x >> 16) * (float)m);
    }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint4 q = lds16_a16(b + 16 + 32 * (e0 >> 6) + (e0 & 16));
        affine16<true>(shr_and(q, (e0 & 32) ? 4 : 0, 0x0F0F0F0Fu), -kTwo23, c, v);
    }
};

template <>
struct Fast<GGML_TYPE_Q5_K> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 176, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int g) { return Fast<GGML_TYPE_Q4_K>::prep(b, g); }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint4 q = lds16_a16(b + 48 + 32 * (e0 >> 6) + (e0 & 16));
        const uint4 h = lds16_a16(b + 16 + (e0 & 16));
        const uint4 lo = shr_and(q, (e0 & 32) ? 4 : 0, 0x0F0F0F0Fu);
        affine16<true>(or_shl(lo, shr_and(h, e0 >> 5, 0x01010101u), 4), -kTwo23, c, v);
    }
};

template <>
struct Fast<GGML_TYPE_Q6_K> {
    static constexpr bool kEnabled = true;
    static constexpr int TILES = 1;
    static constexpr int ELEMS = 256, BYTES = 210, GROUP = 16;
    // group g covers elements 16g..16g+15: half n = g/8, quarter = (g/2)%4, is = g%2 -> scale 8n + is + 2*quarter
    static GGUF_D float2 prep(const uint8_t *b, int g) {
        const int sc = (int8_t)b[192 + 8 * (g >> 3) + (g & 1) + 2 * ((g >> 1) & 3)];
        return make_float2(half_hw(lds_u16(b + 208)) * (float)sc, 0.f);
    }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const int n = e0 >> 7, quarter = (e0 >> 5) & 3, l0 = e0 & 16;
        const uint4 ql = lds16_any(b + 64 * n + 32 * (quarter & 1) + l0);
        const uint4 qh = lds16_any(b + 128 + 32 * n + l0);
        const uint4 lo = shr_and(ql, (quarter & 2) ? 4 : 0, 0x0F0F0F0Fu);
        affine16<false>(or_shl(lo, shr_and(qh, 2 * quarter, 0x03030303u), 4), -(kTwo23 + 32.f), c, v);
    }
};

template <>
struct Fast<GGML_TYPE_Q3_K> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 110, GROUP = 16;
    // group g = scale index of the upstream loop (8n + 2j + half)
    static GGUF_D float2 prep(const uint8_t *b, int g) {
        const uint8_t *s = b + 96;
        const int lo = g < 8 ? (s[g] & 0xF) : (s[g - 8] >> 4);
        const int hi = (s[8 + (g & 3)] >> (2 * (g >> 2))) & 3;
        return make_float2(half_hw(lds_u16(b + 108)) * (float)((lo | (hi << 4)) - 32), 0.f);
    }
    // groups g and g + 8 (g < 8) take the two nibbles of one scale byte and two fields of one high-bits byte
    static GGUF_D void prep_pair(const uint8_t *b, int g, float2 *out) {
        const uint32_t s = b[96 + g], h = (uint32_t)b[104 + (g & 3)] >> (2 * (g >> 2));
        const float d = half_hw(lds_u16(b + 108));
        out[g] = make_float2(d * (float)((int)((s & 0xF) | ((h & 3) << 4)) - 32), 0.f);
        out[g + 8] = make_float2(d * (float)((int)((s >> 4) | (((h >> 4) & 3) << 4)) - 32), 0.f);
    }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const int n = e0 >> 7, j = (e0 >> 5) & 3, r = e0 & 16;
        const uint4 q = lds16_any(b + 32 + 32 * n + r);
        const uint4 hm = lds16_any(b + r);
        // level = low2 + 4*highbit - 4
        affine16<false>(or_shl(shr_and(q, 2 * j, 0x03030303u), shr_and(hm, 4 * n + j, 0x01010101u), 2), -(kTwo23 + 4.f), c, v);
    }
};

template <>
struct Fast<GGML_TYPE_Q2_K> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 84, GROUP = 16;
    static GGUF_D float2 prep(const uint8_t *b, int g) {
        const uint32_t dm = *reinterpret_cast<const uint32_t *>(b + 80);
        const int sc = b[g];
        return make_float2(half_hw(dm & 0xFFFFu) * (float)(sc & 0xF), half_hw(dm >> 16) * (float)(sc >> 4));
    }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint4 q = lds16_a4(b + 16 + 32 * (e0 >> 7) + (e0 & 16));
        affine16<true>(shr_and(q, 2 * ((e0 >> 5) & 3), 0x03030303u), -kTwo23, c, v);
    }
};

// Sixteen-entry byte table lookup for four 4-bit indices at once.  `nibs`: the indices in the low 16
// bits; table entries 0..7 in the bytes of (lo0, lo1), 8..15 in (hi0, hi1).  Two permutes look the low
// three index bits up in either half, a third picks per byte by the index's top bit.
GGUF_D uint32_t lut16x4(uint32_t nibs, uint32_t lo0, uint32_t lo1, uint32_t hi0, uint32_t hi1) {
    const uint32_t sel = nibs & 0x7777u;
    const uint32_t a = __byte_perm(lo0, lo1, sel), b = __byte_perm(hi0, hi1, sel);
    return __byte_perm(a, b, ((nibs >> 1) & 0x4444u) | 0x3210u);
}
// Table of sixteen int8 levels stored with an offset of 128 so that the bytes are unsigned.
struct Lut16 { uint32_t lo0, lo1, hi0, hi1; };
GGUF_HD constexpr uint32_t pack_levels(int a, int b, int c, int d) {
    return (uint32_t)(a + 128) | ((uint32_t)(b + 128) << 8) | ((uint32_t)(c + 128) << 16) | ((uint32_t)(d + 128) << 24);
}
// E2M1 levels times two (code 8, "-0", decodes to 0 like the int8 table entry) and the IQ4 levels.
GGUF_D constexpr Lut16 fp4_lut() { return {pack_levels(0, 1, 2, 3), pack_levels(4, 6, 8, 12), pack_levels(0, -1, -2, -3), pack_levels(-4, -6, -8, -12)}; }
GGUF_D constexpr Lut16 iq4_lut() { return {pack_levels(-127, -104, -83, -65), pack_levels(-49, -35, -22, -10), pack_levels(1, 13, 25, 38),
                           pack_levels(53, 69, 89, 113)}; }

// 16 bytes of packed 4-bit codes, byte j = code(j) | code(j + HALF) << 4, through a level table:
// v[j] = scale * level(code(j)) for j < 16 and v[HALF_OUT + j] for the high nibbles.
// Word k, low half: codes of elements (4k, 4k+H, 4k+1, 4k+H+1); high half: (4k+2, 4k+H+2, 4k+3, 4k+H+3).
template <int WORDS, int HIGH_AT>
GGUF_D void lut_decode(const uint32_t *w, const Lut16 t, float scale, float *v) {
    const float2 nb = make_float2(-(kTwo23 + 128.f), -(kTwo23 + 128.f)), sc = make_float2(scale, scale);
#pragma unroll
    for (int k = 0; k < WORDS; ++k) {
        const uint32_t r0 = lut16x4(w[k], t.lo0, t.lo1, t.hi0, t.hi1), r1 = lut16x4(w[k] >> 16, t.lo0, t.lo1, t.hi0, t.hi1);
        float2 lo01 = make_float2(magic_byte(r0, 0), magic_byte(r0, 2)), hi01 = make_float2(magic_byte(r0, 1), magic_byte(r0, 3));
        float2 lo23 = make_float2(magic_byte(r1, 0), magic_byte(r1, 2)), hi23 = make_float2(magic_byte(r1, 1), magic_byte(r1, 3));
        lo01 = __fmul2_rn(sc, __fadd2_rn(lo01, nb));
        hi01 = __fmul2_rn(sc, __fadd2_rn(hi01, nb));
        lo23 = __fmul2_rn(sc, __fadd2_rn(lo23, nb));
        hi23 = __fmul2_rn(sc, __fadd2_rn(hi23, nb));
        v[4 * k] = lo01.x; v[4 * k + 1] = lo01.y; v[4 * k + 2] = lo23.x; v[4 * k + 3] = lo23.y;
        v[HIGH_AT + 4 * k] = hi01.x; v[HIGH_AT + 4 * k + 1] = hi01.y; v[HIGH_AT + 4 * k + 2] = hi23.x; v[HIGH_AT + 4 * k + 3] = hi23.y;
    }
}

template <>
struct Fast<GGML_TYPE_MXFP4> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 32, BYTES = 17, GROUP = 32, CALL = 32;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(e8m0_half_to_f32(b[0]), 0.f); }
    static GGUF_D void run(const uint8_t *b, int, float2 c, float *v) {
        const uint4 q = lds16_any(b + 1);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        lut_decode<4, 16>(w, fp4_lut(), c.x, v);
    }
};

template <>
struct Fast<GGML_TYPE_NVFP4> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 64, BYTES = 36, GROUP = 16;
    static GGUF_D float2 prep(const uint8_t *b, int g) { return make_float2(ue4m3_half_to_f32(b[g]), 0.f); }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint32_t *p = reinterpret_cast<const uint32_t *>(b + 4 + (e0 >> 4) * 8);
        const uint32_t w[2] = {p[0], p[1]};
        lut_decode<2, 8>(w, fp4_lut(), c.x, v);
    }
};

// upstream dequant.cpp (iq4_nl): y[j] = d * kvalues[qs[j] & 0xf], y[j + 16] = d * kvalues[qs[j] >> 4]
template <>
struct Fast<GGML_TYPE_IQ4_NL> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 32, BYTES = 18, GROUP = 32, CALL = 32;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), 0.f); }
    static GGUF_D void run(const uint8_t *b, int, float2 c, float *v) {
        const uint4 q = lds16_any(b + 2);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        lut_decode<4, 16>(w, iq4_lut(), c.x, v);
    }
};

template <>
struct Fast<GGML_TYPE_IQ4_XS> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 136, GROUP = 32, CALL = 32;
    static GGUF_D float2 prep(const uint8_t *b, int ib) {
        const uint32_t scales_h = lds_u16(b + 2);
        const int ls = ((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (((scales_h >> (2 * ib)) & 3) << 4);
        return make_float2(half_hw(lds_u16(b)) * (float)(ls - 32), 0.f);
    }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint4 q = lds16_a4(b + 8 + (e0 >> 5) * 16);  // 136-byte blocks: 8-byte aligned
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        lut_decode<4, 16>(w, iq4_lut(), c.x, v);
    }
};

// Legacy 4/5-bit types: byte j holds elements j and j + 16.
// Fifth bits of four consecutive elements (bits 0..3 of `bits`) moved to bit 4 of four bytes.
GGUF_D uint32_t spread_bit4(uint32_t bits) { return (((bits & 0xFu) * 0x00204081u) & 0x01010101u) << 4; }

template <bool FIVE, bool HAS_MIN>
GGUF_D void legacy_run(const uint8_t *qs, uint32_t qh, float2 c, float *v) {
    const uint4 q = lds16_any(qs);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    const float neg_bias = -(kTwo23 + (HAS_MIN ? 0.f : (FIVE ? 16.f : 8.f)));
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t lo = w[k] & 0x0F0F0F0Fu, hi = (w[k] >> 4) & 0x0F0F0F0Fu;
        if (FIVE) {
            lo |= spread_bit4(qh >> (4 * k));
            hi |= spread_bit4(qh >> (16 + 4 * k));
        }
        affine4<HAS_MIN>(lo, neg_bias, c, v + 4 * k);
        affine4<HAS_MIN>(hi, neg_bias, c, v + 16 + 4 * k);
    }
}

template <>
struct Fast<GGML_TYPE_Q4_0> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 32, BYTES = 18, GROUP = 32, CALL = 32;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), 0.f); }
    static GGUF_D void run(const uint8_t *b, int, float2 c, float *v) { legacy_run<false, false>(b + 2, 0, c, v); }
};
template <>
struct Fast<GGML_TYPE_Q4_1> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 32, BYTES = 20, GROUP = 32, CALL = 32;
    // x * d + m: affine4 subtracts its second constant
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), -half_hw(lds_u16(b + 2))); }
    static GGUF_D void run(const uint8_t *b, int, float2 c, float *v) { legacy_run<false, true>(b + 4, 0, c, v); }
};
template <>
struct Fast<GGML_TYPE_Q5_0> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 32, BYTES = 22, GROUP = 32, CALL = 32;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), 0.f); }
    static GGUF_D void run(const uint8_t *b, int, float2 c, float *v) {
        legacy_run<true, false>(b + 6, lds_u16(b + 2) | (lds_u16(b + 4) << 16), c, v);
    }
};
template <>
struct Fast<GGML_TYPE_Q5_1> {
    static constexpr bool kEnabled = true;
    static constexpr int TILES = 1;
    static constexpr int ELEMS = 32, BYTES = 24, GROUP = 32, CALL = 32;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), -half_hw(lds_u16(b + 2))); }
    static GGUF_D void run(const uint8_t *b, int, float2 c, float *v) {
        legacy_run<true, true>(b + 8, *reinterpret_cast<const uint32_t *>(b + 4), c, v);
    }
};

// ---- codebook types ----------------------------------------------------------------------------
// unaligned little-endian 32-bit value from a 2-byte aligned shared-memory address
GGUF_D uint32_t lds_u32_a2(const uint8_t *p) { return lds_u16(p) | (lds_u16(p + 2) << 16); }

// A packed codebook entry holds eight 2-bit codes (IQ2, IQ1) or four 3-bit codes (IQ3).  The decoders keep
// every entry already widened to permute selectors (one nibble per coordinate); the levels themselves sit in
// registers and a PRMT looks four of them up at once.  For the IQ2 and IQ3 families the element's sign goes
// into bit 2 of its nibble (IQ2: the permute then reads the level from a table of +levels and -levels) or
// into a second permute that picks between the +level and the -level (IQ3).  The levels are stored with an offset of 128, removed
// together with the 2^23 of the byte-to-float step.  The tables are copied to shared memory by every
// CTA: a gather over a 1-4 KB table costs a few bank conflicts there, one L1 wavefront per touched
// line in global memory.
namespace selectors {
#define GGUF_CODEBOOK(name, count, ...) constexpr uint16_t packed_##name[count] = {__VA_ARGS__};
#include "gguf_codebooks.inc"
#undef GGUF_CODEBOOK
template <class T, int N>
struct Table { T v[N]; };
constexpr uint32_t widen2(uint32_t c) {
    c = (c | (c << 8)) & 0x00FF00FFu;
    c = (c | (c << 4)) & 0x0F0F0F0Fu;
    return (c | (c << 2)) & 0x33333333u;
}
constexpr uint32_t widen3(uint32_t c) {
    c = (c & 0x03Fu) | ((c << 2) & 0x3F00u);
    return (c & 0x0707u) | ((c << 1) & 0x7070u);
}
template <int N>
constexpr Table<uint32_t, N> make2(const uint16_t (&packed)[N]) {
    Table<uint32_t, N> t{};
    for (int i = 0; i < N; ++i) t.v[i] = widen2(packed[i]);
    return t;
}
template <int N>
constexpr Table<uint16_t, N> make3(const uint16_t (&packed)[N]) {
    Table<uint16_t, N> t{};
    for (int i = 0; i < N; ++i) t.v[i] = (uint16_t)widen3(packed[i]);
    return t;
}
// bit j of s (8 bits) -> bit 2 of nibble j
constexpr uint32_t sign_nibbles(uint32_t s) {
    uint32_t x = (s | (s << 12)) & 0x000F000Fu;
    x = (x | (x << 6)) & 0x03030303u;
    return ((x << 2) | (x << 5)) & 0x44444444u;
}
// The sign patterns, ready for use: N = 128 for the formats that store a 7-bit index (the eighth sign makes the
// parity even, upstream libgguf_tables.cpp ksigns_iq2xs), 256 for those that store the byte.  PICK = false: the
// bits to OR into a 2-bit entry's selectors; PICK = true: per half, the selector that picks byte k from the
// +levels (k) or the -levels (4 + k).
template <int N, bool PICK>
constexpr Table<uint32_t, N> make_signs() {
    Table<uint32_t, N> t{};
    for (uint32_t i = 0; i < (uint32_t)N; ++i) {
        uint32_t s = i;
        if (N == 128) {
            uint32_t parity = 0;
            for (int k = 0; k < 7; ++k) parity ^= (i >> k) & 1u;
            s |= parity << 7;
        }
        const uint32_t x = sign_nibbles(s);
        t.v[i] = PICK ? (((x & 0xFFFFu) | 0x3210u) | (((x >> 16) | 0x3210u) << 16)) : x;
    }
    return t;
}
template <class E, int NE, int NS>
struct Tables {
    Table<E, NE> entry;
    Table<uint32_t, NS> signs;
};
}  // namespace selectors
static __device__ __align__(16) const selectors::Tables<uint32_t, 256, 128> k_tab_IQ2XXS = {
    selectors::make2(selectors::packed_IQ2XXS), selectors::make_signs<128, false>()};
static __device__ __align__(16) const selectors::Tables<uint32_t, 512, 128> k_tab_IQ2XS = {
    selectors::make2(selectors::packed_IQ2XS), selectors::make_signs<128, false>()};
static __device__ __align__(16) const selectors::Tables<uint32_t, 1024, 256> k_tab_IQ2S = {
    selectors::make2(selectors::packed_IQ2S), selectors::make_signs<256, false>()};
static __device__ __align__(16) const selectors::Tables<uint16_t, 256, 128> k_tab_IQ3XXS = {
    selectors::make3(selectors::packed_IQ3XXS), selectors::make_signs<128, true>()};
static __device__ __align__(16) const selectors::Tables<uint16_t, 512, 256> k_tab_IQ3S = {
    selectors::make3(selectors::packed_IQ3S), selectors::make_signs<256, true>()};
static __device__ __align__(16) const selectors::Table<uint32_t, 2048> k_tab_IQ1S = selectors::make2(selectors::packed_IQ1S);

// IQ1: v = scale * ((code + 1 - 1) + bias') with bias = -1 -+ 0.125 already holding the -1.  The codes 0..2 enter
// the mantissa of 2^20 in units of 1/8 (table bytes 0, 8, 16), so one subtraction of 2^20 - bias removes the
// magic constant and applies the bias; both are multiples of 1/8 below 2^21, hence exact, as are upstream's two steps.
constexpr uint32_t kIq1Eighths = 0u | (8u << 8) | (16u << 16);
GGUF_D float magic_eighths(uint32_t w, int k) { return __uint_as_float(__byte_perm(w, 0x49800000u, 0x7640u | (uint32_t)k)); }
GGUF_D void emit_iq1(uint32_t sel, float scale, float bias, float *v) {
    const float off = bias - 1048576.f;
    const float2 nb = make_float2(off, off), sc = make_float2(scale, scale);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t levels = __byte_perm(kIq1Eighths, 0, sel >> (16 * h));
        const float2 a = __fmul2_rn(sc, __fadd2_rn(make_float2(magic_eighths(levels, 0), magic_eighths(levels, 1)), nb));
        const float2 b = __fmul2_rn(sc, __fadd2_rn(make_float2(magic_eighths(levels, 2), magic_eighths(levels, 3)), nb));
        v[4 * h] = a.x; v[4 * h + 1] = a.y; v[4 * h + 2] = b.x; v[4 * h + 3] = b.y;
    }
}

constexpr uint32_t biased_levels(int a, int b, int c, int d) {
    return (uint32_t)(128 + a) | ((uint32_t)(128 + b) << 8) | ((uint32_t)(128 + c) << 16) | ((uint32_t)(128 + d) << 24);
}
constexpr uint32_t kIq2Plus = biased_levels(8, 25, 43, 0), kIq2Minus = biased_levels(-8, -25, -43, 0);
constexpr uint32_t kIq3xxsPlus0 = biased_levels(4, 12, 20, 28), kIq3xxsPlus1 = biased_levels(36, 44, 52, 62);
constexpr uint32_t kIq3xxsMinus0 = biased_levels(-4, -12, -20, -28), kIq3xxsMinus1 = biased_levels(-36, -44, -52, -62);
constexpr uint32_t kIq3sPlus0 = biased_levels(1, 3, 5, 7), kIq3sPlus1 = biased_levels(9, 11, 13, 15);
constexpr uint32_t kIq3sMinus0 = biased_levels(-1, -3, -5, -7), kIq3sMinus1 = biased_levels(-9, -11, -13, -15);

// v[0..3] = scale * (byte_k(levels) - 128)
GGUF_D void emit4_biased(uint32_t levels, float scale, float *v) {
    const float2 nb = make_float2(-(kTwo23 + 128.f), -(kTwo23 + 128.f)), sc = make_float2(scale, scale);
    const float2 a = __fmul2_rn(sc, __fadd2_rn(make_float2(magic_byte(levels, 0), magic_byte(levels, 1)), nb));
    const float2 b = __fmul2_rn(sc, __fadd2_rn(make_float2(magic_byte(levels, 2), magic_byte(levels, 3)), nb));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
// Eight values of a 2-bit grid point: sel = the entry's selectors, signs = the sign table's entry.
GGUF_D void emit_signed2(uint32_t sel, uint32_t signs, float scale, float *v) {
    sel |= signs;
    emit4_biased(__byte_perm(kIq2Plus, kIq2Minus, sel), scale, v);
    emit4_biased(__byte_perm(kIq2Plus, kIq2Minus, sel >> 16), scale, v + 4);
}
// Eight values of two 3-bit grid points (four each); pick = the sign table's entry.
GGUF_D void emit_signed3(uint32_t sel_a, uint32_t sel_b, uint32_t pick, uint32_t p0, uint32_t p1, uint32_t m0, uint32_t m1,
                         float scale, float *v) {
    emit4_biased(__byte_perm(__byte_perm(p0, p1, sel_a), __byte_perm(m0, m1, sel_a), pick), scale, v);
    emit4_biased(__byte_perm(__byte_perm(p0, p1, sel_b), __byte_perm(m0, m1, sel_b), pick >> 16), scale, v + 4);
}

// ---- 16-bit outputs by selection -----------------------------------------------------------------------------
// When a group of elements can take only a handful of distinct values (three for IQ1 and TQ1_0), the
// fp16 / bf16 output needs no per-element arithmetic: the candidates are computed once per group with the same fp32
// operations as in the arithmetic path and rounded to the output type once, their low bytes and their high bytes
// are gathered into two "planes", and a codebook entry's nibbles -- one code per element -- are used directly as
// the selector of a byte permute over each plane.  Two more permutes interleave the planes into 16-bit outputs.
// (Tried for IQ3 as well -- eight magnitudes per group, the sign as an XOR on the high-byte plane: 6.0 instead of 7.4
// instructions per element and no faster; those decoders wait for their shared-memory gathers, three per eight
// elements at about 3.4 bank wavefronts each, not for the arithmetic.)
template <class OutT>
GGUF_D uint32_t pack16(float a, float b) {  // a in the low half
    if constexpr (std::is_same<OutT, __half>::value) {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
}
// planes of the patterns packed in p01 (two of them) and p23: lo = their low bytes, hi = their high bytes
GGUF_D void planes4(uint32_t p01, uint32_t p23, uint32_t &lo, uint32_t &hi) {
    lo = __byte_perm(p01, p23, 0x6420u);
    hi = __byte_perm(p01, p23, 0x7531u);
}
// four outputs: nibble j of sel (0..7) picks the pattern of element j from the eight in (lo_a, lo_b) / (hi_a, hi_b)
GGUF_D void select4(uint32_t sel, uint32_t lo_a, uint32_t lo_b, uint32_t hi_a, uint32_t hi_b, uint32_t *w, uint32_t sign_plane = 0u) {
    const uint32_t l = __byte_perm(lo_a, lo_b, sel), h = __byte_perm(hi_a, hi_b, sel) ^ sign_plane;
    w[0] = __byte_perm(l, h, 0x5140u);
    w[1] = __byte_perm(l, h, 0x7362u);
}

// Four sign bits (bit j = element j negative) -> 0x80 in byte j, to be XORed into a plane of high bytes.  The four
// shifted copies the multiplication adds up occupy disjoint bit positions (7 k + j), so nothing carries.
GGUF_D uint32_t sign_plane4(uint32_t s4) { return ((s4 * 0x00204081u) & 0x01010101u) << 7; }

template <>
struct Fast<GGML_TYPE_IQ2_XXS> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 66, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int ib32) {
        const uint32_t aux1 = lds_u32_a2(b + 2 + 8 * ib32 + 4);
        return make_float2(half_hw(lds_u16(b)) * (0.5f + (float)(aux1 >> 28)) * 0.25f, 0.f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ2XXS);
    static GGUF_D const void *table() { return &k_tab_IQ2XXS; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ2XXS) *>(tab);
        const uint8_t *q = b + 2 + 8 * (e0 >> 5);
        const uint32_t aux1 = lds_u32_a2(q + 4);
        const int l = (e0 >> 3) & 3;  // 0 or 2
        const uint32_t pair = lds_u16(q + l);
#pragma unroll
        for (int k = 0; k < 2; ++k)
            emit_signed2(t->entry.v[(pair >> (8 * k)) & 0xFFu], t->signs.v[(aux1 >> (7 * (l + k))) & 127], c.x, v + 8 * k);
    }
    // 16-bit outputs by selection: |value| is one of db * {8, 25, 43}; the sign planes are computed from the sign bits
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ2XXS) *>(tab);
        const uint8_t *q = b + 2 + 8 * (e0 >> 5);
        const uint32_t aux1 = lds_u32_a2(q + 4);
        const int l = (e0 >> 3) & 3;  // 0 or 2
        const uint32_t pair = lds_u16(q + l);
        uint32_t lo, hi;
        planes4(pack16<OutT>(c.x * 8.f, c.x * 25.f), pack16<OutT>(c.x * 43.f, 0.f), lo, hi);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t e = t->entry.v[(pair >> (8 * k)) & 0xFFu];
            const uint32_t sg = iq_signs_from_index((aux1 >> (7 * (l + k))) & 127u);
            select4(e, lo, 0u, hi, 0u, w + 4 * k, sign_plane4(sg & 15u));
            select4(e >> 16, lo, 0u, hi, 0u, w + 4 * k + 2, sign_plane4(sg >> 4));
        }
    }
};

template <>
struct Fast<GGML_TYPE_IQ2_XS> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 74, GROUP = 16;
    static GGUF_D float2 prep(const uint8_t *b, int g16) {
        const int sc = b[66 + (g16 >> 1)];
        return make_float2(half_hw(lds_u16(b)) * (0.5f + (float)((g16 & 1) ? (sc >> 4) : (sc & 0xF))) * 0.25f, 0.f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ2XS);
    static GGUF_D const void *table() { return &k_tab_IQ2XS; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ2XS) *>(tab);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t q = lds_u16(b + 2 + 2 * ((e0 >> 3) + k));
            emit_signed2(t->entry.v[q & 511u], t->signs.v[q >> 9], c.x, v + 8 * k);
        }
    }
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ2XS) *>(tab);
        uint32_t lo, hi;
        planes4(pack16<OutT>(c.x * 8.f, c.x * 25.f), pack16<OutT>(c.x * 43.f, 0.f), lo, hi);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t q = lds_u16(b + 2 + 2 * ((e0 >> 3) + k));
            const uint32_t e = t->entry.v[q & 511u];
            const uint32_t sg = iq_signs_from_index(q >> 9);
            select4(e, lo, 0u, hi, 0u, w + 4 * k, sign_plane4(sg & 15u));
            select4(e >> 16, lo, 0u, hi, 0u, w + 4 * k + 2, sign_plane4(sg >> 4));
        }
    }
};

template <>
struct Fast<GGML_TYPE_IQ2_S> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 82, GROUP = 16;
    static GGUF_D float2 prep(const uint8_t *b, int g16) {
        const int sc = b[74 + (g16 >> 1)];
        return make_float2(half_hw(lds_u16(b)) * (0.5f + (float)((g16 & 1) ? (sc >> 4) : (sc & 0xF))) * 0.25f, 0.f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ2S);
    static GGUF_D const void *table() { return &k_tab_IQ2S; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ2S) *>(tab);
        const int g = e0 >> 3, ib32 = g >> 2;
        const uint32_t qh = b[66 + ib32];
        const uint32_t low = lds_u16(b + 2 + g), signs = lds_u16(b + 2 + 32 + g);  // g is even
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = (g & 3) + k;
            const uint32_t idx = ((low >> (8 * k)) & 0xFFu) | ((qh << (8 - 2 * l)) & 0x300u);
            emit_signed2(t->entry.v[idx], t->signs.v[(signs >> (8 * k)) & 0xFFu], c.x, v + 8 * k);
        }
    }
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ2S) *>(tab);
        const int g = e0 >> 3, ib32 = g >> 2;
        const uint32_t qh = b[66 + ib32];
        const uint32_t low = lds_u16(b + 2 + g), signs = lds_u16(b + 2 + 32 + g);  // g is even
        uint32_t lo, hi;
        planes4(pack16<OutT>(c.x * 8.f, c.x * 25.f), pack16<OutT>(c.x * 43.f, 0.f), lo, hi);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = (g & 3) + k;
            const uint32_t e = t->entry.v[((low >> (8 * k)) & 0xFFu) | ((qh << (8 - 2 * l)) & 0x300u)];
            const uint32_t sg = (signs >> (8 * k)) & 0xFFu;
            select4(e, lo, 0u, hi, 0u, w + 4 * k, sign_plane4(sg & 15u));
            select4(e >> 16, lo, 0u, hi, 0u, w + 4 * k + 2, sign_plane4(sg >> 4));
        }
    }
};

template <>
struct Fast<GGML_TYPE_IQ3_XXS> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 98, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int ib32) {
        const uint32_t aux = lds_u32_a2(b + 2 + 64 + 4 * ib32);
        return make_float2(half_hw(lds_u16(b)) * (0.5f + (float)(aux >> 28)) * 0.5f, 0.f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ3XXS);
    static GGUF_D const void *table() { return &k_tab_IQ3XXS; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ3XXS) *>(tab);
        const int g = e0 >> 3, ib32 = g >> 2;  // g even: grid points 2g .. 2g+3
        const uint32_t aux = lds_u32_a2(b + 2 + 64 + 4 * ib32);
        const uint32_t idx = lds_u32_a2(b + 2 + 2 * g);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t signs = t->signs.v[(aux >> (7 * ((g & 3) + k))) & 127];
            emit_signed3(t->entry.v[(idx >> (16 * k)) & 0xFFu], t->entry.v[(idx >> (16 * k + 8)) & 0xFFu], signs, kIq3xxsPlus0, kIq3xxsPlus1,
                         kIq3xxsMinus0, kIq3xxsMinus1, c.x, v + 8 * k);
        }
    }
    // 16-bit outputs by selection: |value| is one of db * {4, 12, ..., 52, 62} (eight patterns in four planes), the sign
    // an XOR on the plane of high bytes, computed from the sign bits (a table of ready-made planes cost a third
    // shared-memory gather per eight elements and made this path slower than the arithmetic one).
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ3XXS) *>(tab);
        const int g = e0 >> 3, ib32 = g >> 2;  // g even: grid points 2g .. 2g+3
        const uint32_t aux = lds_u32_a2(b + 2 + 64 + 4 * ib32);
        const uint32_t idx = lds_u32_a2(b + 2 + 2 * g);
        uint32_t lo_a, lo_b, hi_a, hi_b;
        planes4(pack16<OutT>(c.x * 4.f, c.x * 12.f), pack16<OutT>(c.x * 20.f, c.x * 28.f), lo_a, hi_a);
        planes4(pack16<OutT>(c.x * 36.f, c.x * 44.f), pack16<OutT>(c.x * 52.f, c.x * 62.f), lo_b, hi_b);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t s = iq_signs_from_index((aux >> (7 * ((g & 3) + k))) & 127u);
            select4(t->entry.v[(idx >> (16 * k)) & 0xFFu], lo_a, lo_b, hi_a, hi_b, w + 4 * k, sign_plane4(s & 15u));
            select4(t->entry.v[(idx >> (16 * k + 8)) & 0xFFu], lo_a, lo_b, hi_a, hi_b, w + 4 * k + 2, sign_plane4(s >> 4));
        }
    }
};

template <>
struct Fast<GGML_TYPE_IQ3_S> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 110, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int ib32) {
        const int sc = b[106 + (ib32 >> 1)];
        return make_float2(half_hw(lds_u16(b)) * (float)(1 + 2 * ((ib32 & 1) ? (sc >> 4) : (sc & 0xF))), 0.f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ3S);
    static GGUF_D const void *table() { return &k_tab_IQ3S; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ3S) *>(tab);
        const int g = e0 >> 3, ib32 = g >> 2;
        const uint32_t qh = b[66 + ib32];
        const uint32_t idx = lds_u32_a2(b + 2 + 2 * g), sg = lds_u16(b + 74 + g);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = (g & 3) + k;
            const uint32_t i1 = ((idx >> (16 * k)) & 0xFFu) | ((qh << (8 - 2 * l)) & 256u);
            const uint32_t i2 = ((idx >> (16 * k + 8)) & 0xFFu) | ((qh << (7 - 2 * l)) & 256u);
            emit_signed3(t->entry.v[i1], t->entry.v[i2], t->signs.v[(sg >> (8 * k)) & 0xFFu], kIq3sPlus0, kIq3sPlus1, kIq3sMinus0, kIq3sMinus1, c.x, v + 8 * k);
        }
    }
    // 16-bit outputs by selection (see IQ3_XXS): |value| is one of db * {1, 3, ..., 15}
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const auto *t = static_cast<const decltype(k_tab_IQ3S) *>(tab);
        const int g = e0 >> 3, ib32 = g >> 2;
        const uint32_t qh = b[66 + ib32];
        const uint32_t idx = lds_u32_a2(b + 2 + 2 * g), sg = lds_u16(b + 74 + g);
        uint32_t lo_a, lo_b, hi_a, hi_b;
        planes4(pack16<OutT>(c.x * 1.f, c.x * 3.f), pack16<OutT>(c.x * 5.f, c.x * 7.f), lo_a, hi_a);
        planes4(pack16<OutT>(c.x * 9.f, c.x * 11.f), pack16<OutT>(c.x * 13.f, c.x * 15.f), lo_b, hi_b);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = (g & 3) + k;
            const uint32_t s = (sg >> (8 * k)) & 0xFFu;
            const uint32_t i1 = ((idx >> (16 * k)) & 0xFFu) | ((qh << (8 - 2 * l)) & 256u);
            const uint32_t i2 = ((idx >> (16 * k + 8)) & 0xFFu) | ((qh << (7 - 2 * l)) & 256u);
            select4(t->entry.v[i1], lo_a, lo_b, hi_a, hi_b, w + 4 * k, sign_plane4(s & 15u));
            select4(t->entry.v[i2], lo_a, lo_b, hi_a, hi_b, w + 4 * k + 2, sign_plane4(s >> 4));
        }
    }
};

// IQ1: value = dl * ((code - 1) + delta), delta = -+0.125; the constant pair holds dl and delta - 1.
template <>
struct Fast<GGML_TYPE_IQ1_S> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 50, GROUP = 32;
    static GGUF_D float2 prep(const uint8_t *b, int ib) {
        const uint32_t qh = lds_u16(b + 34 + 2 * ib);
        return make_float2(half_hw(lds_u16(b)) * (float)(2 * ((qh >> 12) & 7) + 1), (qh & 0x8000u) ? -1.125f : -0.875f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ1S);
    static GGUF_D const void *table() { return &k_tab_IQ1S; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const uint32_t *sel = static_cast<const uint32_t *>(tab);
        const int g = e0 >> 3, ib = g >> 2;
        const uint32_t qh = lds_u16(b + 34 + 2 * ib), low = lds_u16(b + 2 + g);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = (g & 3) + k;
            const uint32_t idx = ((low >> (8 * k)) & 0xFFu) | (((qh >> (3 * l)) & 7u) << 8);
            emit_iq1(sel[idx], c.x, c.y, v + 8 * k);
        }
    }
    // 16-bit outputs: the 32 elements of a group take one of dl * (code + bias), code 0..2
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const uint32_t *sel = static_cast<const uint32_t *>(tab);
        const int g = e0 >> 3, ib = g >> 2;
        const uint32_t qh = lds_u16(b + 34 + 2 * ib), low = lds_u16(b + 2 + g);
        uint32_t lo, hi;
        planes4(pack16<OutT>(c.x * (0.f + c.y), c.x * (1.f + c.y)), pack16<OutT>(c.x * (2.f + c.y), 0.f), lo, hi);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = (g & 3) + k;
            const uint32_t e = sel[((low >> (8 * k)) & 0xFFu) | (((qh >> (3 * l)) & 7u) << 8)];
            select4(e, lo, 0u, hi, 0u, w + 4 * k);
            select4(e >> 16, lo, 0u, hi, 0u, w + 4 * k + 2);
        }
    }
};

template <>
struct Fast<GGML_TYPE_IQ1_M> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 56, GROUP = 16;
    static GGUF_D float2 prep(const uint8_t *b, int g16) {
        const uint32_t s0 = lds_u16(b + 48), s1 = lds_u16(b + 50), s2 = lds_u16(b + 52), s3 = lds_u16(b + 54);
        const uint32_t dbits = (s0 >> 12) | ((s1 >> 8) & 0x00f0u) | ((s2 >> 4) & 0x0f00u) | (s3 & 0xf000u);
        const int ib = g16 >> 1;
        const uint32_t sc = lds_u16(b + 48 + 2 * (ib >> 1));
        return make_float2(half_hw(dbits) * (float)(2 * ((sc >> (6 * (ib & 1) + 3 * (g16 & 1))) & 7) + 1), 0.f);
    }
    // groups g and g + 8 (g < 8): the block scale, scattered over the top nibbles of the four scale words, is put
    // together once for both
    static GGUF_D void prep_pair(const uint8_t *b, int g, float2 *out) {
        const uint32_t s0 = lds_u16(b + 48), s1 = lds_u16(b + 50), s2 = lds_u16(b + 52), s3 = lds_u16(b + 54);
        const float d = half_hw((s0 >> 12) | ((s1 >> 8) & 0x00f0u) | ((s2 >> 4) & 0x0f00u) | (s3 & 0xf000u));
        const int sh = 6 * ((g >> 1) & 1) + 3 * (g & 1);
        const uint32_t a = g < 4 ? s0 : s1, c = g < 4 ? s2 : s3;   // scale word (g / 2) / 2 and the one two words on
        out[g] = make_float2(d * (float)(2 * ((a >> sh) & 7) + 1), 0.f);
        out[g + 8] = make_float2(d * (float)(2 * ((c >> sh) & 7) + 1), 0.f);
    }
    static constexpr int kTableBytes = sizeof(k_tab_IQ1S);
    static GGUF_D const void *table() { return &k_tab_IQ1S; }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v, const void *tab) {
        const uint32_t *sel = static_cast<const uint32_t *>(tab);
        const int g = e0 >> 3;  // even: grid points g, g + 1 share the byte qh[g / 2]
        const uint32_t qh = b[32 + (g >> 1)], low = lds_u16(b + g);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t idx = ((low >> (8 * k)) & 0xFFu) | ((qh << (k ? 4 : 8)) & 0x700u);
            const float bias = (qh & (k ? 0x80u : 0x08u)) ? -1.125f : -0.875f;
            emit_iq1(sel[idx], c.x, bias, v + 8 * k);
        }
    }
    // 16-bit outputs: each grid point's eight elements take one of dl * (code + bias), code 0..2
    template <class OutT>
    static GGUF_D void run16(const uint8_t *b, int e0, float2 c, uint32_t *w, const void *tab) {
        const uint32_t *sel = static_cast<const uint32_t *>(tab);
        const int g = e0 >> 3;
        const uint32_t qh = b[32 + (g >> 1)], low = lds_u16(b + g);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t e = sel[((low >> (8 * k)) & 0xFFu) | ((qh << (k ? 4 : 8)) & 0x700u)];
            const float bias = (qh & (k ? 0x80u : 0x08u)) ? -1.125f : -0.875f;
            uint32_t lo, hi;
            planes4(pack16<OutT>(c.x * (0.f + bias), c.x * (1.f + bias)), pack16<OutT>(c.x * (2.f + bias), 0.f), lo, hi);
            select4(e, lo, 0u, hi, 0u, w + 4 * k);
            select4(e >> 16, lo, 0u, hi, 0u, w + 4 * k + 2);
        }
    }
};

// ---- 1-bit and ternary types --------------------------------------------------------------------
template <>
struct Fast<GGML_TYPE_Q1_0> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 128, BYTES = 18, GROUP = 128;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b)), 0.f); }
    // bit set: d, bit clear: -d
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint32_t clear = ~lds_u16(b + 2 + (e0 >> 3));
        const uint32_t dbits = __float_as_uint(c.x);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(dbits ^ ((clear << (31 - i)) & 0x80000000u));
    }
};

template <>
struct Fast<GGML_TYPE_TQ2_0> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 66, GROUP = 256;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b + 64)), 0.f); }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const uint4 q = lds16_any(b + 32 * (e0 >> 7) + (e0 & 16));
        affine16<false>(shr_and(q, 2 * ((e0 >> 5) & 3), 0x03030303u), -(kTwo23 + 1.f), c, v);
    }
};

// TQ1_0: digit n of a byte is ((byte * 3^n) & 0xFF) * 3 >> 8.  Elements 0..159 take digit e/32 of byte
// e%32, elements 160..239 digit (e-160)/16 of byte 32 + (e-160)%16, elements 240..255 digit (e-240)/4
// of byte 48 + (e-240)%4.  Four bytes at a time: the even and the odd bytes are multiplied in 16-bit
// lanes (255 * 81 < 2^15, so nothing crosses a lane); after the multiplication by 3 (at most 765) the
// digit is the lane's high byte, which the byte-to-float permute picks up directly.
GGUF_D void tq1_emit4(uint32_t w, uint32_t pow3, float2 c, float *v) {
    const uint32_t even = (((w & 0x00FF00FFu) * pow3) & 0x00FF00FFu) * 3u;
    const uint32_t odd = ((((w >> 8) & 0x00FF00FFu) * pow3) & 0x00FF00FFu) * 3u;
    const float2 nb = make_float2(-(kTwo23 + 1.f), -(kTwo23 + 1.f)), sc = make_float2(c.x, c.x);
    const float2 a = __fmul2_rn(sc, __fadd2_rn(make_float2(magic_byte(even, 1), magic_byte(odd, 1)), nb));
    const float2 b = __fmul2_rn(sc, __fadd2_rn(make_float2(magic_byte(even, 3), magic_byte(odd, 3)), nb));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <>
struct Fast<GGML_TYPE_TQ1_0> {
    static constexpr bool kEnabled = true;
    static constexpr int ELEMS = 256, BYTES = 54, GROUP = 256;
    static GGUF_D float2 prep(const uint8_t *b, int) { return make_float2(half_hw(lds_u16(b + 52)), 0.f); }
    static GGUF_D void run(const uint8_t *b, int e0, float2 c, float *v) {
        const bool last = e0 >= 240;
        const int n = e0 < 160 ? e0 >> 5 : (e0 - 160) >> 4;           // digit for the first two regions
        const int at = e0 < 160 ? (e0 & 31) : (last ? 48 : 32);      // first source byte
        const uint32_t p = n == 0 ? 1u : n == 1 ? 3u : n == 2 ? 9u : n == 3 ? 27u : 81u;
        const uint4 q = lds16_any(b + at);  // 54-byte blocks: the 16 bytes stay inside the tile's padding
        const uint32_t w[4] = {q.x, last ? q.x : q.y, last ? q.x : q.z, last ? q.x : q.w};
        const uint32_t pw[4] = {last ? 1u : p, last ? 3u : p, last ? 9u : p, last ? 27u : p};
#pragma unroll
        for (int i = 0; i < 4; ++i) tq1_emit4(w[i], pw[i], c, v + 4 * i);
    }
};

// ---------------------------------------------------------------------------------------------
template <class OutT>
struct OutPack;

template <>
struct OutPack<float> {
    static GGUF_D void store8(float *dst, const float *v, bool aligned) {
        if (aligned) {
            __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
            __stcs(reinterpret_cast<float4 *>(dst) + 1, make_float4(v[4], v[5], v[6], v[7]));
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = v[i];
        }
    }
};

template <>
struct OutPack<__half> {
    static GGUF_D void store8(__half *dst, const float *v, bool aligned) {
        if (aligned) {
            uint4 u;
            __half2 h;
            h = __floats2half2_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t *>(&h);
            h = __floats2half2_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t *>(&h);
            h = __floats2half2_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t *>(&h);
            h = __floats2half2_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t *>(&h);
            __stcs(reinterpret_cast<uint4 *>(dst), u);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = __float2half_rn(v[i]);
        }
    }
};

template <>
struct OutPack<__nv_bfloat16> {
    static GGUF_D void store8(__nv_bfloat16 *dst, const float *v, bool aligned) {
        if (aligned) {
            uint4 u;
            __nv_bfloat162 h;
            h = __floats2bfloat162_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t *>(&h);
            h = __floats2bfloat162_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t *>(&h);
            h = __floats2bfloat162_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t *>(&h);
            h = __floats2bfloat162_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t *>(&h);
            __stcs(reinterpret_cast<uint4 *>(dst), u);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = __float2bfloat16_rn(v[i]);
        }
    }
};

constexpr int kThreads = 256;
constexpr int kRunsPerThread = 4;                       // runs of 8 elements each thread decodes
constexpr int kTileElems = kThreads * 8 * kRunsPerThread;  // 8192 elements per CTA

template <int TYPE, class OutT>
__global__ void __launch_bounds__(kThreads) dequant_tile_kernel(const uint8_t *__restrict__ src, OutT *__restrict__ dst,
                                                               int64_t nblocks, int dst_aligned) {
    using D = Decoder<TYPE>;
    constexpr int TILE_BLOCKS = kTileElems / D::ELEMS;
    constexpr int TILE_BYTES = TILE_BLOCKS * D::BYTES;
    __shared__ __align__(16) uint8_t tile[TILE_BYTES + 32];

    const int64_t b0 = (int64_t)blockIdx.x * TILE_BLOCKS;
    const int nb = (int)(nblocks - b0 < TILE_BLOCKS ? nblocks - b0 : TILE_BLOCKS);
    const uint8_t *gsrc = src + b0 * D::BYTES;
    const int nbytes = nb * D::BYTES;
    // Stage the 16-byte aligned span [gsrc - mis, gsrc + nbytes) rounded up to 16.  The extra
    // bytes share a 16-byte granule with bytes of the tile, so they are in the same page.
    const int mis = (int)(reinterpret_cast<uintptr_t>(gsrc) & 15);
    const uint4 *g16 = reinterpret_cast<const uint4 *>(gsrc - mis);
    const int nvec = (mis + nbytes + 15) >> 4;
    uint4 *s16 = reinterpret_cast<uint4 *>(tile);
    grid_dependents_may_launch();
    grid_dependency_wait();
    for (int i = threadIdx.x; i < nvec; i += kThreads) s16[i] = __ldcs(g16 + i);
    __syncthreads();

    const uint8_t *blocks = tile + mis;
    OutT *out = dst + b0 * D::ELEMS;
    const int nruns = nb * (D::ELEMS / 8);
#pragma unroll
    for (int u = 0; u < kRunsPerThread; ++u) {
        const int run = u * kThreads + threadIdx.x;
        if (run < nruns) {
            const int e = run * 8;
            const int blk = e / D::ELEMS;
            float v[8];
            D::run(blocks + blk * D::BYTES, e - blk * D::ELEMS, v);
            OutPack<OutT>::store8(out + e, v, dst_aligned != 0);
        }
    }
}

// 256-bit streaming store of 8 words (sm_100).
GGUF_D void st_v8(void *p, const uint32_t (&w)[8]) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}
template <class OutT>
GGUF_D void store16(OutT *dst, const float *v) {
    uint32_t w[8];
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(v[8 * h + i]);
            st_v8(reinterpret_cast<float *>(dst) + 8 * h, w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if constexpr (std::is_same<OutT, __half>::value) {
                const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t *>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t *>(&h);
            }
        }
        st_v8(dst, w);
    }
}

// Decoders that derive the constants of two groups from the same bytes provide prep_pair(block, g, out)
// for groups g and g + GROUPS_PER_BLOCK / 2.
template <class D, class = void>
struct HasPrepPair : std::false_type {};
template <class D>
struct HasPrepPair<D, std::void_t<decltype(&D::prep_pair)>> : std::true_type {};

// Decoders that look codebook entries up provide kTableBytes / table(): the kernel copies the table to
// shared memory and hands it to run() as a fifth argument.
template <class D, class = void>
struct TableBytes { static constexpr int value = 0; };
template <class D>
struct TableBytes<D, std::void_t<decltype(D::kTableBytes)>> { static constexpr int value = D::kTableBytes; };

// Decoders with a selection path for 16-bit outputs provide run16<OutT>(block, e0, constants, words, table), which
// writes CALL16 (default: the arithmetic path's call size) packed outputs.
template <class D, class OutT, class = void>
struct HasRun16 : std::false_type {};
template <class D, class OutT>
struct HasRun16<D, OutT, std::void_t<decltype(&D::template run16<OutT>)>> : std::true_type {};
template <class D, class = void>
struct Call16Elems { static constexpr int value = CallElems<D>::value; };
template <class D>
struct Call16Elems<D, decltype((void)D::CALL16)> { static constexpr int value = D::CALL16; };

// Tiles a CTA of the fast kernel decodes: two (16384 elements), both tiles' loads issued before the first is decoded,
// so that the launch of the CTA, the wait for the previous kernel and, for the codebook types, the copy of the table
// to shared memory (1-8 KB, as much as half of the 16 KB of 16-bit output a tile has) are paid once for both.
// Measured on 14336x4096 -> fp16 against one tile per CTA: the codebook types gain 3-14 points of the copy bandwidth
// (IQ3_S 0.89 -> 0.95, IQ1_M 0.88 -> 0.93), IQ4_NL 0.87 -> 0.95, MXFP4 0.88 -> 0.95, Q3_K 0.90 -> 0.94, Q5_K 0.95 -> 0.97;
// the three types with the most encoded bytes per element lose 1-2 points and keep one tile (they set TILES = 1).
// Four tiles per CTA are slower again for nearly every type (0.80-0.92): the staged tiles and constants then take
// enough shared memory to cost resident CTAs.
template <class D, class = void>
struct TilesPerCta { static constexpr int value = 2; };
template <class D>
struct TilesPerCta<D, decltype((void)D::TILES)> { static constexpr int value = D::TILES; };

template <int TYPE, class OutT>
__global__ void __launch_bounds__(kThreads, 8) dequant_fast_kernel(const uint8_t *__restrict__ src, OutT *__restrict__ dst,
                                                               int64_t nblocks) {
    using D = Fast<TYPE>;
    constexpr int TILES = TilesPerCta<D>::value;
    constexpr int TILE_BLOCKS = kTileElems / D::ELEMS;
    constexpr int TILE_BYTES = TILE_BLOCKS * D::BYTES;
    constexpr int TILE_VECS = (TILE_BYTES + 15) / 16;
    constexpr int TILE_GROUPS = kTileElems / D::GROUP;
    constexpr int GROUPS_PER_BLOCK = D::ELEMS / D::GROUP;
    static_assert(TILE_BYTES % 16 == 0, "every tile starts on a 16-byte boundary");
    __shared__ __align__(16) uint8_t tiles[TILES][TILE_VECS * 16 + 32];
    __shared__ float2 all_consts[TILES][TILE_GROUPS];

    const int tid = threadIdx.x;
    const int64_t first_block = (int64_t)blockIdx.x * TILES * TILE_BLOCKS;
    constexpr int TABLE_BYTES = TableBytes<D>::value;
    static_assert(TABLE_BYTES % 16 == 0, "the table moves as 16-byte vectors");
    __shared__ __align__(16) uint8_t table[TABLE_BYTES ? TABLE_BYTES : 16];
    grid_dependents_may_launch();
    if constexpr (TABLE_BYTES > 0) {  // constant data: does not wait for the previous kernel
        const uint4 *g = static_cast<const uint4 *>(D::table());
#pragma unroll
        for (int k = 0; k < (TABLE_BYTES / 16 + kThreads - 1) / kThreads; ++k) {
            const int i = k * kThreads + tid;
            if (i < TABLE_BYTES / 16) reinterpret_cast<uint4 *>(table)[i] = __ldg(g + i);
        }
    }
    grid_dependency_wait();
    int nbs[TILES];
#pragma unroll
    for (int ti = 0; ti < TILES; ++ti) {
        const int64_t b0 = first_block + (int64_t)ti * TILE_BLOCKS;
        nbs[ti] = b0 >= nblocks ? 0 : (int)(nblocks - b0 < TILE_BLOCKS ? nblocks - b0 : TILE_BLOCKS);
        const uint4 *g16 = reinterpret_cast<const uint4 *>(src + b0 * D::BYTES);  // 16-byte aligned by contract
        const int nvec = (nbs[ti] * D::BYTES + 15) >> 4;
        uint4 *s16 = reinterpret_cast<uint4 *>(tiles[ti]);
#pragma unroll
        for (int k = 0; k < (TILE_VECS + kThreads - 1) / kThreads; ++k) {
            const int i = k * kThreads + tid;
            if (i < nvec) s16[i] = __ldcs(g16 + i);
        }
    }
    __syncthreads();
#pragma unroll
    for (int ti = 0; ti < TILES; ++ti) {
        const uint8_t *tile = tiles[ti];
        float2 *consts = all_consts[ti];
        const int nb = nbs[ti];
        if constexpr (HasPrepPair<D>::value) {
            constexpr int PAIRS = GROUPS_PER_BLOCK / 2;
#pragma unroll
            for (int k = 0; k < (TILE_GROUPS / 2 + kThreads - 1) / kThreads; ++k) {
                const int p = k * kThreads + tid;
                const int blk = p / PAIRS;
                if (blk < nb) D::prep_pair(tile + blk * D::BYTES, p % PAIRS, consts + blk * GROUPS_PER_BLOCK);
            }
        } else {
#pragma unroll
            for (int k = 0; k < (TILE_GROUPS + kThreads - 1) / kThreads; ++k) {
                const int g = k * kThreads + tid;
                const int blk = g / GROUPS_PER_BLOCK;
                if (blk < nb) consts[g] = D::prep(tile + blk * D::BYTES, g % GROUPS_PER_BLOCK);
            }
        }
    }
    __syncthreads();
    // call c = u*kThreads + tid: position inside the block (e0) does not depend on u
    constexpr bool SELECT16 = sizeof(OutT) == 2 && HasRun16<D, OutT>::value;
    constexpr int CALL = SELECT16 ? Call16Elems<D>::value : CallElems<D>::value;
    constexpr int CALLS_PER_BLOCK = D::ELEMS / CALL;
    constexpr int CALLS_PER_THREAD = kTileElems / CALL / kThreads;  // 2 or 1
    static_assert(kThreads % CALLS_PER_BLOCK == 0, "a thread keeps its position inside the block across iterations");
    const int e0 = (tid % CALLS_PER_BLOCK) * CALL;
    const int blk0 = tid / CALLS_PER_BLOCK;
#pragma unroll
    for (int ti = 0; ti < TILES; ++ti) {
        const int nb = nbs[ti];
        OutT *out = dst + (first_block + (int64_t)ti * TILE_BLOCKS) * D::ELEMS + (int64_t)blk0 * D::ELEMS + e0;
        const uint8_t *bp = tiles[ti] + blk0 * D::BYTES;
        const float2 *cp = all_consts[ti] + (blk0 * D::ELEMS + e0) / D::GROUP;
#pragma unroll
        for (int u = 0; u < CALLS_PER_THREAD; ++u) {
            constexpr int BLOCK_STEP = kThreads / CALLS_PER_BLOCK;
            if constexpr (SELECT16) {
                if (blk0 + u * BLOCK_STEP < nb) {
                    uint32_t w[CALL / 2];
                    D::template run16<OutT>(bp + u * BLOCK_STEP * D::BYTES, e0, cp[u * BLOCK_STEP * GROUPS_PER_BLOCK], w, table);
#pragma unroll
                    for (int h = 0; h < CALL / 16; ++h)
                        st_v8(out + (int64_t)u * BLOCK_STEP * D::ELEMS + 16 * h, *reinterpret_cast<const uint32_t(*)[8]>(w + 8 * h));
                }
            } else if (blk0 + u * BLOCK_STEP < nb) {
                float v[CALL];
                if constexpr (TABLE_BYTES > 0) D::run(bp + u * BLOCK_STEP * D::BYTES, e0, cp[u * BLOCK_STEP * GROUPS_PER_BLOCK], v, table);
                else D::run(bp + u * BLOCK_STEP * D::BYTES, e0, cp[u * BLOCK_STEP * GROUPS_PER_BLOCK], v);
#pragma unroll
                for (int h = 0; h < CALL / 16; ++h) store16<OutT>(out + (int64_t)u * BLOCK_STEP * D::ELEMS + 16 * h, v + 16 * h);
            }
        }
    }
}

// ---- decoding by selection: 16-bit outputs of the types with at most four distinct values per group ----------
// A TQ1_0 element is d * (digit - 1) with digit in {0, 1, 2}: a block has three possible outputs.  For fp16 / bf16
// output they are computed once per block (the same fp32 products as in the arithmetic path, rounded to the output
// type once) and every element becomes a byte permute that picks one of the three 16-bit patterns; no
// per-element floating point, no conversion.  The permute selectors come from a 256-entry table: for each byte
// value, its five base-3 digits (upstream dequant.cpp:345-383: digit n of byte v is ((v * 3^n mod 256) * 3) >> 8)
// already written as selector bytes (low nibble 2t, high nibble 2t + 1 pick the two bytes of pattern t).
// A thread owns eight consecutive bytes of a block and writes, digit by digit, the eight elements each digit
// yields (they sit 32, 16 or 4 apart in the block); a thread that owned consecutive elements would need a
// different digit of sixteen different bytes instead.
namespace tq1 {
constexpr uint32_t digit(uint32_t v, int n) {
    uint32_t q = v;
    for (int i = 0; i < n; ++i) q = (q * 3u) & 0xFFu;
    return (q * 3u) >> 8;
}
struct SelectorTable { uint2 v[256]; };
constexpr SelectorTable make_table() {
    SelectorTable t{};
    for (uint32_t v = 0; v < 256; ++v) {
        uint32_t lo = 0;
        for (int n = 0; n < 4; ++n) lo |= (34u * digit(v, n) + 16u) << (8 * n);
        t.v[v].x = lo;
        t.v[v].y = 34u * digit(v, 4) + 16u;
    }
    return t;
}
}  // namespace tq1
static __device__ __align__(16) const tq1::SelectorTable k_tq1_selectors = tq1::make_table();

constexpr int kTq1Threads = 224;  // 128 tasks over bytes 0..31, 64 over bytes 32..47, 32 over bytes 48..51 of 32 blocks

// The tasks store their 16-byte runs straight to global memory (a warp's store covers 64-byte pieces, 512 bytes apart).
// Gathering the tile's outputs in shared memory first, so that every store fills whole 128-byte lines, was measured and
// is slower (0.63 against 0.84 of the copy bandwidth): the extra pass through shared memory costs more than the
// half-filled lines.
constexpr int kTq1TilesPerCta = 2;  // the table copy, the launch and the wait for the previous kernel are paid once for two tiles

template <class OutT>
__global__ void __launch_bounds__(kTq1Threads, 6) dequant_tq1_select_kernel(const uint8_t *__restrict__ src, OutT *__restrict__ dst,
                                                                           int64_t nblocks) {
    static_assert(sizeof(OutT) == 2, "selection works on 16-bit patterns");
    constexpr int TILE_BLOCKS = kTileElems / 256, BYTES = 54;
    constexpr int TILE_VECS = (TILE_BLOCKS * BYTES + 15) / 16;
    __shared__ __align__(16) uint8_t tiles[kTq1TilesPerCta][TILE_VECS * 16 + 16];
    __shared__ __align__(16) uint2 table[256];
    const int tid = threadIdx.x;
    grid_dependents_may_launch();
    {   // constant data: does not wait for the previous kernel
        const uint4 *g = reinterpret_cast<const uint4 *>(&k_tq1_selectors);
        if (tid < 128) reinterpret_cast<uint4 *>(table)[tid] = __ldg(g + tid);
    }
    grid_dependency_wait();
    const int64_t first_block = (int64_t)blockIdx.x * kTq1TilesPerCta * TILE_BLOCKS;
#pragma unroll
    for (int ti = 0; ti < kTq1TilesPerCta; ++ti) {   // both tiles' loads are in flight before the first is decoded
        const int64_t b0 = first_block + ti * TILE_BLOCKS;
        const int nb = b0 >= nblocks ? 0 : (int)(nblocks - b0 < TILE_BLOCKS ? nblocks - b0 : TILE_BLOCKS);
        const uint4 *g16 = reinterpret_cast<const uint4 *>(src + b0 * BYTES);  // 16-byte aligned by contract (1728 bytes per tile)
        const int nvec = (nb * BYTES + 15) >> 4;
        if (tid < nvec) reinterpret_cast<uint4 *>(tiles[ti])[tid] = __ldcs(g16 + tid);  // at most 108 vectors
    }
    __syncthreads();

    // task -> block, first byte, element offset of digit 0, element stride between digits
    int blk, at, first, stride;
    if (tid < 128) { blk = tid >> 2; at = 8 * (tid & 3); first = at; stride = 32; }
    else if (tid < 192) { blk = (tid - 128) >> 1; at = 32 + 8 * (tid & 1); first = 160 + 8 * (tid & 1); stride = 16; }
    else { blk = tid - 192; at = 48; first = 240; stride = 4; }
#pragma unroll 1
    for (int ti = 0; ti < kTq1TilesPerCta; ++ti) {
        const int64_t b0 = first_block + ti * TILE_BLOCKS;
        if (b0 + blk >= nblocks) break;
        const uint8_t *b = tiles[ti] + blk * BYTES;
        // the block's three outputs as 16-bit patterns
        const float d = half_hw(lds_u16(b + 52));
        const uint32_t lut_a = pack16<OutT>(d * -1.0f, d * 0.0f), lut_b = pack16<OutT>(d * 1.0f, d * 1.0f);
        OutT *out = dst + (b0 + blk) * 256 + first;
        const uint32_t w0 = lds_u32_a2(b + at);
        if (tid >= 192) {
            // four bytes, four digits each: elements 240 + 4 n + j, sixteen consecutive outputs
            uint2 e[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) e[i] = table[(w0 >> (8 * i)) & 0xFFu];
            uint32_t w[8];
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const uint32_t pick = ((4u + n) << 4) | (uint32_t)n;
                w[2 * n] = __byte_perm(lut_a, lut_b, __byte_perm(e[0].x, e[1].x, pick));
                w[2 * n + 1] = __byte_perm(lut_a, lut_b, __byte_perm(e[2].x, e[3].x, pick));
            }
            st_v8(out, w);
            continue;
        }
        const uint32_t w1 = lds_u32_a2(b + at + 4);
        uint2 e[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            e[i] = table[(w0 >> (8 * i)) & 0xFFu];
            e[4 + i] = table[(w1 >> (8 * i)) & 0xFFu];
        }
#pragma unroll
        for (int n = 0; n < 5; ++n) {
            uint4 o;
            if (n < 4) {
                const uint32_t pick = ((4u + n) << 4) | (uint32_t)n;
                o.x = __byte_perm(lut_a, lut_b, __byte_perm(e[0].x, e[1].x, pick));
                o.y = __byte_perm(lut_a, lut_b, __byte_perm(e[2].x, e[3].x, pick));
                o.z = __byte_perm(lut_a, lut_b, __byte_perm(e[4].x, e[5].x, pick));
                o.w = __byte_perm(lut_a, lut_b, __byte_perm(e[6].x, e[7].x, pick));
            } else {
                o.x = __byte_perm(lut_a, lut_b, __byte_perm(e[0].y, e[1].y, 0x40u));
                o.y = __byte_perm(lut_a, lut_b, __byte_perm(e[2].y, e[3].y, 0x40u));
                o.z = __byte_perm(lut_a, lut_b, __byte_perm(e[4].y, e[5].y, 0x40u));
                o.w = __byte_perm(lut_a, lut_b, __byte_perm(e[6].y, e[7].y, 0x40u));
            }
            __stcs(reinterpret_cast<uint4 *>(out + n * stride), o);
        }
    }
}

template <int TYPE, class OutT>
cudaError_t launch_typed(const void *src, void *dst, int64_t nelems, cudaStream_t stream) {
    using D = Decoder<TYPE>;
    const int64_t nblocks = nelems / D::ELEMS;
    constexpr int TILE_BLOCKS = kTileElems / D::ELEMS;
    const int64_t grid = (nblocks + TILE_BLOCKS - 1) / TILE_BLOCKS;
    if (grid <= 0) return cudaSuccess;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    const int aligned = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    if constexpr (TYPE == GGML_TYPE_TQ1_0 && sizeof(OutT) == 2) {
        if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            const cudaError_t launched = launch_overlapped(dequant_tq1_select_kernel<OutT>, (unsigned)((grid + kTq1TilesPerCta - 1) / kTq1TilesPerCta), kTq1Threads, stream,
                                                           static_cast<const uint8_t *>(src), static_cast<OutT *>(dst), nblocks);
            count_launch();
            return launched != cudaSuccess ? launched : cudaGetLastError();
        }
    }
    if constexpr (Fast<TYPE>::kEnabled) {
        if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            constexpr int TILES = TilesPerCta<Fast<TYPE>>::value;
            const cudaError_t launched = launch_overlapped(dequant_fast_kernel<TYPE, OutT>, (unsigned)((grid + TILES - 1) / TILES), kThreads, stream,
                                                           static_cast<const uint8_t *>(src), static_cast<OutT *>(dst), nblocks);
            count_launch();
            return launched != cudaSuccess ? launched : cudaGetLastError();
        }
    }
    const cudaError_t launched = launch_overlapped(dequant_tile_kernel<TYPE, OutT>, (unsigned)grid, kThreads, stream,
                                                   static_cast<const uint8_t *>(src), static_cast<OutT *>(dst), nblocks, aligned);
    count_launch();
    return launched != cudaSuccess ? launched : cudaGetLastError();
}

// bf16 rows whose length is not a multiple of 8: scalar tail handled by a tiny kernel.
template <class OutT>
__global__ void bf16_tail_kernel(const uint16_t *src, OutT *dst, int64_t begin, int64_t n) {
    const int64_t i = begin + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < n) {
        const float f = bits_to_f32((uint32_t)src[i] << 16);
        if constexpr (sizeof(OutT) == 4) dst[i] = f;
        else if constexpr (std::is_same<OutT, __half>::value) dst[i] = __float2half_rn(f);
        else dst[i] = __float2bfloat16_rn(f);
    }
}

template <class OutT>
cudaError_t launch_for_out(int type, const void *src, void *dst, int64_t nelems, cudaStream_t stream) {
    switch (type) {
#define GGUF_CASE(T) case T: return launch_typed<T, OutT>(src, dst, nelems, stream);
        GGUF_CASE(GGML_TYPE_Q4_0) GGUF_CASE(GGML_TYPE_Q4_1) GGUF_CASE(GGML_TYPE_Q5_0) GGUF_CASE(GGML_TYPE_Q5_1)
        GGUF_CASE(GGML_TYPE_Q8_0) GGUF_CASE(GGML_TYPE_Q1_0) GGUF_CASE(GGML_TYPE_MXFP4) GGUF_CASE(GGML_TYPE_NVFP4)
        GGUF_CASE(GGML_TYPE_Q2_K) GGUF_CASE(GGML_TYPE_Q3_K) GGUF_CASE(GGML_TYPE_Q4_K) GGUF_CASE(GGML_TYPE_Q5_K)
        GGUF_CASE(GGML_TYPE_Q6_K) GGUF_CASE(GGML_TYPE_TQ1_0) GGUF_CASE(GGML_TYPE_TQ2_0) GGUF_CASE(GGML_TYPE_IQ2_XXS)
        GGUF_CASE(GGML_TYPE_IQ2_XS) GGUF_CASE(GGML_TYPE_IQ2_S) GGUF_CASE(GGML_TYPE_IQ3_XXS) GGUF_CASE(GGML_TYPE_IQ3_S)
        GGUF_CASE(GGML_TYPE_IQ1_S) GGUF_CASE(GGML_TYPE_IQ1_M) GGUF_CASE(GGML_TYPE_IQ4_NL) GGUF_CASE(GGML_TYPE_IQ4_XS)
#undef GGUF_CASE
        case GGML_TYPE_BF16: {
            const int64_t main_elems = nelems & ~(int64_t)7;
            cudaError_t err = launch_typed<GGML_TYPE_BF16, OutT>(src, dst, main_elems, stream);
            if (err != cudaSuccess) return err;
            if (main_elems < nelems) {
                bf16_tail_kernel<OutT><<<1, 8, 0, stream>>>(static_cast<const uint16_t *>(src), static_cast<OutT *>(dst),
                                                           main_elems, nelems);
                count_launch();
                err = cudaGetLastError();
            }
            return err;
        }
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_dequantize(int type, const void *src, void *dst, int64_t nelems, int out_dtype, cudaStream_t stream) {
    switch (out_dtype) {
        case 0: return launch_for_out<float>(type, src, dst, nelems, stream);
        case 1: return launch_for_out<__half>(type, src, dst, nelems, stream);
        case 2: return launch_for_out<__nv_bfloat16>(type, src, dst, nelems, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gguf
