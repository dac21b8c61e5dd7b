/*
 * TEST INFRASTRUCTURE -- see gguf_oracle.h.  Plain C11, single-threaded, no FMA contraction.
 *
 * Each function restates one upstream routine; the comment above it names the upstream file and
 * lines it follows.  Arithmetic is written in the same order as upstream because the encoded
 * bytes depend on fp32 rounding of every intermediate.
 */
#include "gguf_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256
#define IMIN(a, b) ((a) < (b) ? (a) : (b))
#define IMAX(a, b) ((a) > (b) ? (a) : (b))

enum {
    T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11,
    T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19,
    T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23, T_IQ1_M = 29, T_BF16 = 30, T_TQ1_0 = 34,
    T_TQ2_0 = 35, T_MXFP4 = 39, T_NVFP4 = 40, T_Q1_0 = 41
};

/* ------------------------------------------------------------------------------------------- */
/* codebooks (wire-format constants, packed 2 or 3 bits per coordinate) */
#define GGUF_CODEBOOK(name, count, ...) static const uint16_t CB_##name[count] = {__VA_ARGS__};
#include "../libgguf_b200/csrc/gguf_codebooks.inc"
#undef GGUF_CODEBOOK

/* upstream libgguf_tables.cpp: kvalues_iq4nl, kvalues_mxfp4 */
static const int8_t IQ4NL_VALUES[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static const int8_t FP4_VALUES[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

static void block_geometry(int type, int *elems, int *bytes) {
    int e = 0, b = 0;
    switch (type) {
        case T_Q4_0: e = 32; b = 18; break;   case T_Q4_1: e = 32; b = 20; break;
        case T_Q5_0: e = 32; b = 22; break;   case T_Q5_1: e = 32; b = 24; break;
        case T_Q8_0: e = 32; b = 34; break;   case T_Q1_0: e = 128; b = 18; break;
        case T_MXFP4: e = 32; b = 17; break;  case T_NVFP4: e = 64; b = 36; break;
        case T_Q2_K: e = 256; b = 84; break;  case T_Q3_K: e = 256; b = 110; break;
        case T_Q4_K: e = 256; b = 144; break; case T_Q5_K: e = 256; b = 176; break;
        case T_Q6_K: e = 256; b = 210; break; case T_TQ1_0: e = 256; b = 54; break;
        case T_TQ2_0: e = 256; b = 66; break; case T_IQ2_XXS: e = 256; b = 66; break;
        case T_IQ2_XS: e = 256; b = 74; break; case T_IQ2_S: e = 256; b = 82; break;
        case T_IQ3_XXS: e = 256; b = 98; break; case T_IQ3_S: e = 256; b = 110; break;
        case T_IQ1_S: e = 256; b = 50; break; case T_IQ1_M: e = 256; b = 56; break;
        case T_IQ4_NL: e = 32; b = 18; break; case T_IQ4_XS: e = 256; b = 136; break;
        default: break;
    }
    *elems = e;
    *bytes = b;
}

size_t gguf_oracle_row_size(int type, int64_t n) {
    if (n <= 0) return 0;
    if (type == T_F32) return (size_t)n * 4;
    if (type == T_F16 || type == T_BF16) return (size_t)n * 2;
    int e, b;
    block_geometry(type, &e, &b);
    if (e == 0 || n % e != 0) return 0;
    return (size_t)(n / e) * (size_t)b;
}

int gguf_oracle_quantize_requires_imatrix(int type) { return type == T_IQ2_XXS || type == T_IQ2_XS || type == T_IQ1_S; }

/* ------------------------------------------------------------------------------------------- */
/* scalar conversions */
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static uint32_t rd32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
static void wr16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
static void wr32(uint8_t *p, uint32_t v) { wr16(p, (uint16_t)v); wr16(p + 2, (uint16_t)(v >> 16)); }

/* upstream libgguf_common.h:28-50 */
static float h2f(uint16_t h) {
    const uint32_t w = (uint32_t)h << 16, sign = w & 0x80000000u, two_w = w + w;
    const float normalized = u2f((two_w >> 4) + (0xE0u << 23)) * 0x1.0p-112f;
    const float denormalized = u2f((two_w >> 17) | (126u << 23)) - 0.5f;
    return u2f(sign | (two_w < (1u << 27) ? f2u(denormalized) : f2u(normalized)));
}

/* upstream libgguf_common.h:52-78 */
static uint16_t f2h(float f) {
    float base = (fabsf(f) * 0x1.0p+112f) * 0x1.0p-110f;
    const uint32_t w = f2u(f), shl1_w = w + w, sign = w & 0x80000000u;
    uint32_t bias = shl1_w & 0xFF000000u;
    if (bias < 0x71000000u) bias = 0x71000000u;
    base = u2f((bias >> 1) + 0x07800000u) + base;
    const uint32_t bits = f2u(base);
    const uint32_t nonsign = ((bits >> 13) & 0x7C00u) + (bits & 0x0FFFu);
    return (uint16_t)((sign >> 16) | (shl1_w > 0xFF000000u ? 0x7E00u : nonsign));
}

/* upstream libgguf_common.h:280-296 */
static uint16_t f2bf(float s) {
    const uint32_t i = f2u(s);
    if ((i & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((i >> 16) | 64);
    return (uint16_t)((i + (0x7fffu + ((i >> 16) & 1))) >> 16);
}

/* upstream libgguf_common.h:124-145 */
static float e8m0_half(uint8_t x) { return u2f(x < 2 ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23)); }

/* upstream libgguf_common.h:152-171 */
static float ue4m3_half(uint8_t x) {
    if (x == 0 || x == 0x7F) return 0.0f;
    const int exp = (x >> 3) & 0xF, man = x & 7;
    const float raw = exp == 0 ? ldexpf((float)man, -9) : ldexpf(1.0f + (float)man / 8.0f, exp - 7);
    return raw * 0.5f;
}

/* upstream libgguf_common.h:173-220 */
static uint8_t f2ue4m3(float x) {
    if (!(x > 0.0f)) return 0;
    if (x > 448.0f) x = 448.0f;
    const uint32_t bits = f2u(x);
    const int fexp = (int)((bits >> 23) & 0xFF) - 127, fman = (bits >> 20) & 7;
    int e = fexp + 7;
    if (e <= 0) {
        int man = (int)(x * 512.0f + 0.5f);
        if (man > 7) man = 7;
        return man < 1 ? 0 : (uint8_t)man;
    }
    if (e >= 15) return 0x7E;
    int m = fman + (int)((bits >> 19) & 1);
    if (m > 7) { m = 0; if (++e >= 15) return 0x7E; }
    return (uint8_t)((e << 3) | m);
}

/* upstream libgguf_common.h:337-344 */
static int nearest_int(float v) { return (int)(f2u(v + 12582912.f) & 0x007fffffu) - 0x00400000; }

/* upstream libgguf_common.h:301-317 */
static int best_index_int8(const int8_t *val, float x) {
    if (x <= val[0]) return 0;
    if (x >= val[15]) return 15;
    int ml = 0, mu = 15;
    while (mu - ml > 1) { const int mav = (ml + mu) / 2; if (x < val[mav]) mu = mav; else ml = mav; }
    return x - val[mu - 1] < val[mu] - x ? mu - 1 : mu;
}

/* upstream libgguf_common.h:321-335 */
static int best_index_fp4(float x, float e) {
    int best = 0;
    float best_err = fabsf(FP4_VALUES[0] * e - x);
    for (int i = 1; i < 16; ++i) {
        const float err = fabsf(FP4_VALUES[i] * e - x);
        if (err < best_err) { best = i; best_err = err; }
    }
    return best;
}

/* upstream libgguf_common.h:672-684 */
static void scale_min_k4(int j, const uint8_t *q, int *d, int *m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

/* ------------------------------------------------------------------------------------------- */
/* decoders: one block -> `elems` floats.  upstream csrc/dequant/dequant.cpp (line refs per case) */
static int iq2_byte(int c) { static const int v[4] = {8, 25, 43, 0}; return v[c]; }
static int iq3xxs_byte(int c) { static const int v[8] = {4, 12, 20, 28, 36, 44, 52, 62}; return v[c]; }
static uint32_t signs7(uint32_t i) { return i | ((uint32_t)(__builtin_popcount(i) & 1) << 7); }

static void emit_iq2(float *y, uint16_t code, uint32_t signs, float db) {
    for (int j = 0; j < 8; ++j) y[j] = db * (float)iq2_byte((code >> (2 * j)) & 3) * ((signs >> j) & 1 ? -1.f : 1.f);
}

static void decode_block(int type, const uint8_t *b, float *y) {
    switch (type) {
        case T_Q8_0: { /* :120-134 */
            const float d = h2f(rd16(b));
            for (int j = 0; j < 32; ++j) y[j] = (int8_t)b[2 + j] * d;
        } break;
        case T_Q4_0: { /* :21-35 */
            const float d = h2f(rd16(b));
            for (int j = 0; j < 16; ++j) { y[j] = ((b[2 + j] & 0xF) - 8) * d; y[j + 16] = ((b[2 + j] >> 4) - 8) * d; }
        } break;
        case T_Q4_1: { /* :37-52 */
            const float d = h2f(rd16(b)), m = h2f(rd16(b + 2));
            for (int j = 0; j < 16; ++j) { y[j] = (b[4 + j] & 0xF) * d + m; y[j + 16] = (b[4 + j] >> 4) * d + m; }
        } break;
        case T_Q5_0: { /* :54-76 */
            const float d = h2f(rd16(b));
            const uint32_t qh = rd32(b + 2);
            for (int j = 0; j < 16; ++j) {
                const int x0 = ((b[6 + j] & 0xF) | (((qh >> j) & 1) << 4)) - 16;
                const int x1 = ((b[6 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4)) - 16;
                y[j] = x0 * d; y[j + 16] = x1 * d;
            }
        } break;
        case T_Q5_1: { /* :78-101 */
            const float d = h2f(rd16(b)), m = h2f(rd16(b + 2));
            const uint32_t qh = rd32(b + 4);
            for (int j = 0; j < 16; ++j) {
                const int x0 = (b[8 + j] & 0xF) | (((qh >> j) & 1) << 4);
                const int x1 = (b[8 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
                y[j] = x0 * d + m; y[j + 16] = x1 * d + m;
            }
        } break;
        case T_Q1_0: { /* :6-19 */
            const float d = h2f(rd16(b));
            for (int j = 0; j < 128; ++j) y[j] = (b[2 + j / 8] >> (j % 8)) & 1 ? d : -d;
        } break;
        case T_MXFP4: { /* :136-154 */
            const float d = e8m0_half(b[0]);
            for (int j = 0; j < 16; ++j) { y[j] = FP4_VALUES[b[1 + j] & 0xF] * d; y[j + 16] = FP4_VALUES[b[1 + j] >> 4] * d; }
        } break;
        case T_NVFP4: { /* :156-179 */
            for (int s = 0; s < 4; ++s) {
                const float d = ue4m3_half(b[s]);
                for (int j = 0; j < 8; ++j) {
                    y[16 * s + j] = FP4_VALUES[b[4 + 8 * s + j] & 0xF] * d;
                    y[16 * s + j + 8] = FP4_VALUES[b[4 + 8 * s + j] >> 4] * d;
                }
            }
        } break;
        case T_Q2_K: { /* :181-211 */
            const float d = h2f(rd16(b + 80)), mn = h2f(rd16(b + 82));
            const uint8_t *q = b + 16;
            int is = 0;
            for (int n = 0; n < 2; ++n, q += 32)
                for (int j = 0; j < 4; ++j)
                    for (int half = 0; half < 2; ++half) {
                        const uint8_t sc = b[is++];
                        const float dl = d * (sc & 0xF), ml = mn * (sc >> 4);
                        for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l + 16 * half] >> (2 * j)) & 3)) - ml;
                    }
        } break;
        case T_Q3_K: { /* :213-261 */
            const float d_all = h2f(rd16(b + 108));
            const uint8_t *q = b + 32, *hm = b, *s = b + 96;
            int8_t scales[16];
            for (int i = 0; i < 16; ++i) {
                const int lo = i < 8 ? (s[i] & 0xF) : (s[i - 8] >> 4);
                scales[i] = (int8_t)(lo | (((s[8 + (i & 3)] >> (2 * (i >> 2))) & 3) << 4));
            }
            int is = 0;
            uint8_t m = 1;
            for (int n = 0; n < 2; ++n, q += 32)
                for (int j = 0; j < 4; ++j, m <<= 1)
                    for (int half = 0; half < 2; ++half) {
                        const float dl = d_all * (scales[is++] - 32);
                        for (int l = 0; l < 16; ++l)
                            *y++ = dl * ((int8_t)((q[l + 16 * half] >> (2 * j)) & 3) - ((hm[l + 16 * half] & m) ? 0 : 4));
                    }
        } break;
        case T_Q4_K: { /* :263-285 */
            const float d = h2f(rd16(b)), mn = h2f(rd16(b + 2));
            const uint8_t *q = b + 16;
            for (int j = 0; j < 4; ++j, q += 32) {
                int sc, m;
                scale_min_k4(2 * j, b + 4, &sc, &m);
                const float d1 = d * sc, m1 = mn * m;
                scale_min_k4(2 * j + 1, b + 4, &sc, &m);
                const float d2 = d * sc, m2 = mn * m;
                for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 0xF) - m1;
                for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
            }
        } break;
        case T_Q5_K: { /* :287-312 */
            const float d = h2f(rd16(b)), mn = h2f(rd16(b + 2));
            const uint8_t *ql = b + 48, *qh = b + 16;
            uint8_t u1 = 1, u2 = 2;
            for (int j = 0; j < 4; ++j, ql += 32, u1 <<= 2, u2 <<= 2) {
                int sc, m;
                scale_min_k4(2 * j, b + 4, &sc, &m);
                const float d1 = d * sc, m1 = mn * m;
                scale_min_k4(2 * j + 1, b + 4, &sc, &m);
                const float d2 = d * sc, m2 = mn * m;
                for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 0xF) + (qh[l] & u1 ? 16 : 0)) - m1;
                for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + (qh[l] & u2 ? 16 : 0)) - m2;
            }
        } break;
        case T_Q6_K: { /* :314-343 */
            const float d = h2f(rd16(b + 208));
            const uint8_t *ql = b, *qh = b + 128;
            const int8_t *sc = (const int8_t *)(b + 192);
            for (int n = 0; n < 2; ++n, y += 128, ql += 64, qh += 32, sc += 8)
                for (int l = 0; l < 32; ++l) {
                    const int is = l / 16;
                    const int8_t q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                    const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                    const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    y[l] = d * sc[is] * q1; y[l + 32] = d * sc[is + 2] * q2;
                    y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4;
                }
        } break;
        case T_TQ1_0: { /* :345-383 */
            static const uint8_t pow3[5] = {1, 3, 9, 27, 81};
            const float d = h2f(rd16(b + 52));
            for (int n = 0; n < 5; ++n) for (int m = 0; m < 32; ++m) { const uint8_t q = (uint8_t)(b[m] * pow3[n]); *y++ = (float)((((uint16_t)q * 3) >> 8) - 1) * d; }
            for (int n = 0; n < 5; ++n) for (int m = 0; m < 16; ++m) { const uint8_t q = (uint8_t)(b[32 + m] * pow3[n]); *y++ = (float)((((uint16_t)q * 3) >> 8) - 1) * d; }
            for (int n = 0; n < 4; ++n) for (int j = 0; j < 4; ++j) { const uint8_t q = (uint8_t)(b[48 + j] * pow3[n]); *y++ = (float)((((uint16_t)q * 3) >> 8) - 1) * d; }
        } break;
        case T_TQ2_0: { /* :385-401 */
            const float d = h2f(rd16(b + 64));
            for (int j = 0; j < 64; j += 32) for (int l = 0; l < 4; ++l) for (int m = 0; m < 32; ++m) *y++ = (float)(((b[j + m] >> (2 * l)) & 3) - 1) * d;
        } break;
        case T_IQ2_XXS: { /* :403-427 */
            const float d = h2f(rd16(b));
            for (int ib = 0; ib < 8; ++ib) {
                const uint8_t *q = b + 2 + 8 * ib;
                const uint32_t aux = rd32(q + 4);
                const float db = d * (0.5f + (aux >> 28)) * 0.25f;
                for (int l = 0; l < 4; ++l, y += 8) emit_iq2(y, CB_IQ2XXS[q[l]], signs7((aux >> (7 * l)) & 127), db);
            }
        } break;
        case T_IQ2_XS: { /* :429-452 */
            const float d = h2f(rd16(b));
            for (int ib = 0; ib < 8; ++ib) {
                const float db0 = d * (0.5f + (b[66 + ib] & 0xF)) * 0.25f, db1 = d * (0.5f + (b[66 + ib] >> 4)) * 0.25f;
                for (int l = 0; l < 4; ++l, y += 8) {
                    const uint16_t q = rd16(b + 2 + 2 * (4 * ib + l));
                    emit_iq2(y, CB_IQ2XS[q & 511], signs7(q >> 9), l < 2 ? db0 : db1);
                }
            }
        } break;
        case T_IQ2_S: { /* :454-482 */
            const float d = h2f(rd16(b));
            for (int ib = 0; ib < 8; ++ib) {
                const float db0 = d * (0.5f + (b[74 + ib] & 0xF)) * 0.25f, db1 = d * (0.5f + (b[74 + ib] >> 4)) * 0.25f;
                for (int l = 0; l < 4; ++l, y += 8) {
                    const int g = 4 * ib + l;
                    emit_iq2(y, CB_IQ2S[b[2 + g] | ((b[66 + ib] << (8 - 2 * l)) & 0x300)], b[34 + g], l < 2 ? db0 : db1);
                }
            }
        } break;
        case T_IQ3_XXS: { /* :484-512 */
            const float d = h2f(rd16(b));
            for (int ib = 0; ib < 8; ++ib) {
                const uint32_t aux = rd32(b + 66 + 4 * ib);
                const float db = d * (0.5f + (aux >> 28)) * 0.5f;
                for (int l = 0; l < 4; ++l, y += 8) {
                    const uint32_t signs = signs7((aux >> (7 * l)) & 127);
                    const uint16_t c1 = CB_IQ3XXS[b[2 + 8 * ib + 2 * l]], c2 = CB_IQ3XXS[b[2 + 8 * ib + 2 * l + 1]];
                    for (int j = 0; j < 4; ++j) {
                        y[j] = db * (float)iq3xxs_byte((c1 >> (3 * j)) & 7) * ((signs >> j) & 1 ? -1.f : 1.f);
                        y[j + 4] = db * (float)iq3xxs_byte((c2 >> (3 * j)) & 7) * ((signs >> (j + 4)) & 1 ? -1.f : 1.f);
                    }
                }
            }
        } break;
        case T_IQ3_S: { /* :630-669 */
            const float d = h2f(rd16(b));
            for (int ib = 0; ib < 8; ++ib) {
                const int sc = b[106 + ib / 2];
                const float db = d * (1 + 2 * (ib & 1 ? sc >> 4 : sc & 0xF));
                const uint32_t qh = b[66 + ib];
                for (int l = 0; l < 4; ++l, y += 8) {
                    const int g = 4 * ib + l;
                    const uint16_t c1 = CB_IQ3S[b[2 + 2 * g] | ((qh << (8 - 2 * l)) & 256)];
                    const uint16_t c2 = CB_IQ3S[b[2 + 2 * g + 1] | ((qh << (7 - 2 * l)) & 256)];
                    const uint32_t signs = b[74 + g];
                    for (int j = 0; j < 4; ++j) {
                        y[j] = db * (float)(2 * ((c1 >> (3 * j)) & 7) + 1) * ((signs >> j) & 1 ? -1.f : 1.f);
                        y[j + 4] = db * (float)(2 * ((c2 >> (3 * j)) & 7) + 1) * ((signs >> (j + 4)) & 1 ? -1.f : 1.f);
                    }
                }
            }
        } break;
        case T_IQ1_S: { /* :514-538 */
            const float d = h2f(rd16(b));
            for (int ib = 0; ib < 8; ++ib) {
                const uint32_t qh = rd16(b + 34 + 2 * ib);
                const float dl = d * (2 * ((qh >> 12) & 7) + 1);
                const float delta = qh & 0x8000 ? -0.125f : 0.125f;
                for (int l = 0; l < 4; ++l, y += 8) {
                    const uint16_t code = CB_IQ1S[b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
                    for (int j = 0; j < 8; ++j) y[j] = dl * ((float)((int)((code >> (2 * j)) & 3) - 1) + delta);
                }
            }
        } break;
        case T_IQ1_M: { /* :540-587 */
            const uint32_t s0 = rd16(b + 48), s1 = rd16(b + 50), s2 = rd16(b + 52), s3 = rd16(b + 54);
            const float d = h2f((uint16_t)((s0 >> 12) | ((s1 >> 8) & 0x00f0) | ((s2 >> 4) & 0x0f00) | (s3 & 0xf000)));
            for (int ib = 0; ib < 8; ++ib) {
                const uint32_t sc = rd16(b + 48 + 2 * (ib / 2));
                const float dl1 = d * (2 * ((sc >> (6 * (ib % 2) + 0)) & 7) + 1), dl2 = d * (2 * ((sc >> (6 * (ib % 2) + 3)) & 7) + 1);
                for (int l = 0; l < 4; ++l, y += 8) {
                    const uint32_t qh = b[32 + 2 * ib + l / 2];
                    const uint16_t code = CB_IQ1S[b[4 * ib + l] | ((qh << (l & 1 ? 4 : 8)) & 0x700)];
                    const float delta = qh & (l & 1 ? 0x80 : 0x08) ? -0.125f : 0.125f;
                    for (int j = 0; j < 8; ++j) y[j] = (l < 2 ? dl1 : dl2) * ((float)((int)((code >> (2 * j)) & 3) - 1) + delta);
                }
            }
        } break;
        case T_IQ4_NL: { /* :589-603 */
            const float d = h2f(rd16(b));
            for (int j = 0; j < 16; ++j) { y[j] = d * IQ4NL_VALUES[b[2 + j] & 0xF]; y[j + 16] = d * IQ4NL_VALUES[b[2 + j] >> 4]; }
        } break;
        case T_IQ4_XS: { /* :605-628 */
            const float d = h2f(rd16(b));
            const uint32_t sh = rd16(b + 2);
            for (int ib = 0; ib < 8; ++ib, y += 32) {
                const int ls = ((b[4 + ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
                const float dl = d * (ls - 32);
                for (int j = 0; j < 16; ++j) { y[j] = dl * IQ4NL_VALUES[b[8 + 16 * ib + j] & 0xF]; y[j + 16] = dl * IQ4NL_VALUES[b[8 + 16 * ib + j] >> 4]; }
            }
        } break;
        default: break;
    }
}

size_t gguf_oracle_dequantize_chunk(int type, const void *src, float *dst, int64_t start, int64_t nrows, int64_t n) {
    if (nrows <= 0) return 0;
    int e, b;
    block_geometry(type, &e, &b);
    const size_t rs = gguf_oracle_row_size(type, n);
    if (e == 0 || rs == 0 || n <= 0 || start < 0 || start % n != 0) return 0;
    const uint8_t *in = (const uint8_t *)src + (size_t)(start / n) * rs;
    float *out = dst + start;
    const int64_t nb = nrows * n / e;
    for (int64_t i = 0; i < nb; ++i) decode_block(type, in + i * b, out + i * e);
    return (size_t)nrows * (size_t)n * 4;
}

/* ------------------------------------------------------------------------------------------- */
/* scale searches */

/* upstream libgguf_common.h:398-491 (make_qx_quants), rmse_type 1 only (the value every caller
 * on the row path passes). qw may be NULL (then w = x*x). */
static float make_qx_quants(int n, int nmax, const float *x, int8_t *L, const float *qw) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) { const float ax = fabsf(x[i]); if (ax > amax) { amax = ax; max = x[i]; } }
    if (amax < 1e-15f) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
    float iscale = -nmax / max;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        l = IMAX(-nmax, IMIN(nmax - 1, l));
        L[i] = (int8_t)(l + nmax);
        const float w = qw ? qw[i] : x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(nmax + 0.1f * is) / max;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale * x[i]);
            l = IMAX(-nmax, IMIN(nmax - 1, l));
            const float w = qw ? qw[i] : x[i] * x[i];
            sumlx += w * x[i] * l;
            suml2 += w * l * l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) { const int l = nearest_int(iscale * x[i]); L[i] = (int8_t)(nmax + IMAX(-nmax, IMIN(nmax - 1, l))); }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

/* upstream libgguf_common.h:493-572 (make_q3_quants with do_rmse = true) */
static float make_q3_quants(int n, int nmax, const float *x, int8_t *L) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) { const float ax = fabsf(x[i]); if (ax > amax) { amax = ax; max = x[i]; } }
    if (amax < 1e-15f) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
    const float iscale = -nmax / max;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        l = IMAX(-nmax, IMIN(nmax - 1, l));
        L[i] = (int8_t)l;
        const float w = x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float w = x[i] * x[i];
            float slx = sumlx - w * x[i] * L[i];
            if (slx > 0) {
                float sl2 = suml2 - w * L[i] * L[i];
                int new_l = nearest_int(x[i] * sl2 / slx);
                new_l = IMAX(-nmax, IMIN(nmax - 1, new_l));
                if (new_l != L[i]) {
                    slx += w * x[i] * new_l;
                    sl2 += w * new_l * new_l;
                    if (sl2 > 0 && slx * slx * suml2 > sumlx * sumlx * sl2) { L[i] = (int8_t)new_l; sumlx = slx; suml2 = sl2; ++n_changed; }
                }
            }
        }
        if (!n_changed) break;
    }
    for (int i = 0; i < n; ++i) L[i] = (int8_t)(L[i] + nmax);
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

/* upstream libgguf_common.h:574-670 (make_qkx2_quants) and :688-785 (make_qkx3_quants): with
 * explicit weights the two routines perform the same arithmetic. */
static float make_qkx_quants(int n, int nmax, const float *x, const float *w, uint8_t *L, float *the_min, uint8_t *Laux,
                             float rmin, float rdelta, int nstep, int use_mad) {
    float min = x[0], max = x[0], sum_w = w[0], sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        sum_w += w[i];
        sum_x += w[i] * x[i];
    }
    if (min > 0) min = 0;
    if (max == min) { for (int i = 0; i < n; ++i) L[i] = 0; *the_min = -min; return 0.f; }
    float iscale = nmax / (max - min);
    float scale = 1 / iscale;
    float best_error = 0;
    for (int i = 0; i < n; ++i) {
        const int l = nearest_int(iscale * (x[i] - min));
        L[i] = (uint8_t)IMAX(0, IMIN(nmax, l));
        float diff = scale * L[i] + min - x[i];
        diff = use_mad ? fabsf(diff) : diff * diff;
        best_error += w[i] * diff;
    }
    if (nstep < 1) { *the_min = -min; return scale; }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * is + nmax) / (max - min);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale * (x[i] - min));
            l = IMAX(0, IMIN(nmax, l));
            Laux[i] = (uint8_t)l;
            sum_l += w[i] * l;
            sum_l2 += w[i] * l * l;
            sum_xl += w[i] * l * x[i];
        }
        const float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0) { this_min = 0; this_scale = sum_xl / sum_l2; }
            float cur_error = 0;
            for (int i = 0; i < n; ++i) {
                float diff = this_scale * Laux[i] + this_min - x[i];
                diff = use_mad ? fabsf(diff) : diff * diff;
                cur_error += w[i] * diff;
            }
            if (cur_error < best_error) {
                memcpy(L, Laux, (size_t)n);
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

/* upstream libgguf_common.h:787-880 (make_qp_quants) */
static float make_qp_quants(int n, int nmax, const float *x, uint8_t *L, const float *qw) {
    float max = 0;
    for (int i = 0; i < n; ++i) max = max > x[i] ? max : x[i];
    if (max < 1e-15f) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
    float iscale = nmax / max;
    for (int i = 0; i < n; ++i) L[i] = (uint8_t)nearest_int(iscale * x[i]);
    const float scale = 1 / iscale;
    float best_mse = 0;
    for (int i = 0; i < n; ++i) { const float diff = x[i] - scale * L[i]; best_mse += qw[i] * diff * diff; }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        const float iscale_is = (0.1f * is + nmax) / max, scale_is = 1 / iscale_is;
        float mse = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale_is * x[i]);
            l = IMIN(nmax, l);
            const float diff = x[i] - scale_is * l;
            mse += qw[i] * diff * diff;
        }
        if (mse < best_mse) { best_mse = mse; iscale = iscale_is; }
    }
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        l = IMIN(nmax, l);
        L[i] = (uint8_t)l;
        sumlx += qw[i] * x[i] * l;
        suml2 += qw[i] * l * l;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float w = qw[i];
            float slx = sumlx - w * x[i] * L[i];
            float sl2 = suml2 - w * L[i] * L[i];
            if (slx > 0 && sl2 > 0) {
                int new_l = nearest_int(x[i] * sl2 / slx);
                new_l = IMIN(nmax, new_l);
                if (new_l != L[i]) {
                    slx += w * x[i] * new_l;
                    sl2 += w * new_l * new_l;
                    if (slx * slx * suml2 > sumlx * sumlx * sl2) { L[i] = (uint8_t)new_l; sumlx = slx; suml2 = sl2; ++n_changed; }
                }
            }
        }
        if (!n_changed) break;
    }
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

/* ------------------------------------------------------------------------------------------- */
/* quantizers over k consecutive elements (no imatrix) */

/* upstream q8_0.cpp:16-43 */
static void quant_q8_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i, x += 32, y += 34) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) { const float a = fabsf(x[j]); amax = amax > a ? amax : a; }
        const float d = amax / 127, id = d ? 1.0f / d : 0.0f;
        wr16(y, f2h(d));
        for (int j = 0; j < 32; ++j) y[2 + j] = (uint8_t)(int8_t)roundf(x[j] * id);
    }
}

static void pack_q5(uint8_t *qs, uint8_t *qh_out, const uint8_t *v) {
    uint32_t qh = 0;
    for (int j = 0; j < 16; ++j) {
        qs[j] = (uint8_t)((v[j] & 0x0F) | ((v[j + 16] & 0x0F) << 4));
        qh |= ((v[j] & 0x10u) >> 4) << j;
        qh |= ((v[j + 16] & 0x10u) >> 4) << (j + 16);
    }
    wr32(qh_out, qh);
}

/* upstream q4_0.cpp:16-58, q5_0.cpp:18-65 */
static void quant_q4_0_q5_0(const float *x, uint8_t *y, int64_t k, int five) {
    const int bytes = five ? 22 : 18;
    for (int64_t i = 0; i < k / 32; ++i, x += 32, y += bytes) {
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < 32; ++j) if (amax < fabsf(x[j])) { amax = fabsf(x[j]); max = x[j]; }
        const float d = max / (five ? -16 : -8), id = d ? 1.0f / d : 0.0f;
        wr16(y, f2h(d));
        uint8_t v[32];
        for (int j = 0; j < 32; ++j) {
            const int8_t q = (int8_t)(x[j] * id + (five ? 16.5f : 8.5f));
            v[j] = (uint8_t)IMIN(five ? 31 : 15, q);
        }
        if (five) pack_q5(y + 6, y + 2, v);
        else for (int j = 0; j < 16; ++j) y[2 + j] = (uint8_t)(v[j] | (v[j + 16] << 4));
    }
}

/* upstream q4_1.cpp:16-57, q5_1.cpp:18-68 */
static void quant_q4_1_q5_1(const float *x, uint8_t *y, int64_t k, int five) {
    const int bytes = five ? 24 : 20;
    for (int64_t i = 0; i < k / 32; ++i, x += 32, y += bytes) {
        float min = 3.402823466e+38f, max = -3.402823466e+38f;
        for (int j = 0; j < 32; ++j) { if (x[j] < min) min = x[j]; if (x[j] > max) max = x[j]; }
        const float d = (max - min) / (five ? 31 : 15), id = d ? 1.0f / d : 0.0f;
        wr16(y, f2h(d));
        wr16(y + 2, f2h(min));
        uint8_t v[32];
        for (int j = 0; j < 32; ++j) {
            const float t = (x[j] - min) * id + 0.5f;
            v[j] = five ? (uint8_t)t : (uint8_t)IMIN(15, (int8_t)t);
        }
        if (five) pack_q5(y + 8, y + 4, v);
        else for (int j = 0; j < 16; ++j) y[4 + j] = (uint8_t)(v[j] | (v[j + 16] << 4));
    }
}

/* upstream q1_0.cpp:16-55 */
static void quant_q1_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t i = 0; i < k / 128; ++i, x += 128, y += 18) {
        float sum_abs = 0.0f;
        for (int j = 0; j < 128; ++j) sum_abs += fabsf(x[j]);
        wr16(y, f2h(sum_abs / 128));
        memset(y + 2, 0, 16);
        for (int j = 0; j < 128; ++j) if (x[j] >= 0.0f) y[2 + j / 8] |= (uint8_t)(1 << (j % 8));
    }
}

/* upstream mxfp4.cpp:17-54 */
static void quant_mxfp4(const float *x, uint8_t *y, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i, x += 32, y += 17) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) if (amax < fabsf(x[j])) amax = fabsf(x[j]);
        const uint8_t e = amax > 0.0f ? (uint8_t)(floorf(log2f(amax)) - 2 + 127) : 0;
        const float d = e8m0_half(e);
        y[0] = e;
        for (int j = 0; j < 16; ++j) y[1 + j] = (uint8_t)(best_index_fp4(x[j], d) | (best_index_fp4(x[j + 16], d) << 4));
    }
}

/* upstream nvfp4.cpp:16-55 */
static void quant_nvfp4(const float *x, uint8_t *y, int64_t k) {
    for (int64_t i = 0; i < k / 64; ++i, x += 64, y += 36)
        for (int s = 0; s < 4; ++s) {
            const float *xb = x + 16 * s;
            float amax = 0.0f;
            for (int j = 0; j < 16; ++j) if (amax < fabsf(xb[j])) amax = fabsf(xb[j]);
            const uint8_t ue = f2ue4m3(amax / 6.0f);
            y[s] = ue;
            const float d = ue4m3_half(ue);
            for (int j = 0; j < 8; ++j) y[4 + 8 * s + j] = (uint8_t)(best_index_fp4(xb[j], d) | (best_index_fp4(xb[j + 8], d) << 4));
        }
}

static uint8_t trits5(const float *x, int stride, int count, float id) {
    uint8_t q = 0;
    for (int n = 0; n < count; ++n) { q = (uint8_t)(q * 3); q = (uint8_t)(q + (int)lroundf(x[n * stride] * id) + 1); }
    return q;
}

/* upstream tq1_0.cpp:16-98, tq2_0.cpp:16-53 */
static void quant_ternary(const float *x, uint8_t *y, int64_t k, int tq1) {
    const int bytes = tq1 ? 54 : 66;
    for (int64_t i = 0; i < k / 256; ++i, x += 256, y += bytes) {
        float amax = 0.0f;
        for (int j = 0; j < 256; ++j) { const float a = fabsf(x[j]); amax = amax > a ? amax : a; }
        const float d = amax, id = d ? 1.0f / d : 0.0f;
        if (tq1) {
            for (int m = 0; m < 32; ++m) { const uint8_t q = trits5(x + m, 32, 5, id); y[m] = (uint8_t)(((uint16_t)q * 256 + 242) / 243); }
            for (int m = 0; m < 16; ++m) { const uint8_t q = trits5(x + 160 + m, 16, 5, id); y[32 + m] = (uint8_t)(((uint16_t)q * 256 + 242) / 243); }
            for (int j = 0; j < 4; ++j) {
                uint8_t q = trits5(x + 240 + j, 4, 4, id);
                q = (uint8_t)(q * 3);
                y[48 + j] = (uint8_t)(((uint16_t)q * 256 + 242) / 243);
            }
            wr16(y + 52, f2h(d));
        } else {
            for (int j = 0; j < 2; ++j)
                for (int m = 0; m < 32; ++m) {
                    uint8_t q = 0;
                    for (int n = 0; n < 4; ++n) q = (uint8_t)(q + ((((int)lroundf(x[128 * j + m + 32 * n] * id) + 1) & 3) << (2 * n)));
                    y[32 * j + m] = q;
                }
            wr16(y + 64, f2h(d));
        }
    }
}

/* ------------------------------------------------------------------------------------------- */
/* K-quants: one super-block.  qw = importance weights for this super-block or NULL. */

static void pack_scales_k4(uint8_t *scales, const uint8_t *ls, const uint8_t *lm) {
    memset(scales, 0, 12);
    for (int j = 0; j < 8; ++j) {
        if (j < 4) { scales[j] = ls[j]; scales[j + 4] = lm[j]; }
        else {
            scales[j + 4] = (uint8_t)((ls[j] & 0xF) | ((lm[j] & 0xF) << 4));
            scales[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
            scales[j] |= (uint8_t)((lm[j] >> 4) << 6);
        }
    }
}

/* upstream q4_k.cpp:18-110 / :162-251 and q5_k.cpp:18-124 / :187-301 */
static void quant_q4k_q5k_block(const float *x, uint8_t *y, const float *qw, int five) {
    const int nmax = five ? 31 : 15;
    uint8_t L[256], Laux[32], ls[8], lm[8];
    float weights[32], mins[8], scales[8], sw[8];
    float dblock, mblock;
    if (!qw) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 8; ++j) {
            float sum_x2 = 0;
            for (int l = 0; l < 32; ++l) sum_x2 += x[32 * j + l] * x[32 * j + l];
            const float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; ++l) weights[l] = av_x + fabsf(x[32 * j + l]);
            scales[j] = five ? make_qkx_quants(32, 31, x + 32 * j, weights, L + 32 * j, &mins[j], Laux, -0.5f, 0.1f, 15, 0)
                             : make_qkx_quants(32, 15, x + 32 * j, weights, L + 32 * j, &mins[j], Laux, -1.f, 0.1f, 20, 0);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        const float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f, inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        for (int j = 0; j < 8; ++j) {
            uint8_t a = (uint8_t)nearest_int(inv_scale * scales[j]), b = (uint8_t)nearest_int(inv_min * mins[j]);
            ls[j] = a < 63 ? a : 63;
            lm[j] = b < 63 ? b : 63;
        }
        dblock = max_scale / 63.f;
        mblock = max_min / 63.f;
    } else {
        float sum_x2 = 0;
        for (int l = 0; l < 256; ++l) sum_x2 += x[l] * x[l];
        const float sigma2 = 2 * sum_x2 / QK_K;
        for (int j = 0; j < 8; ++j) {
            for (int l = 0; l < 32; ++l) weights[l] = qw[32 * j + l] * sqrtf(sigma2 + x[32 * j + l] * x[32 * j + l]);
            float sumw = 0;
            for (int l = 0; l < 32; ++l) sumw += weights[l];
            sw[j] = sumw;
            scales[j] = make_qkx_quants(32, nmax, x + 32 * j, weights, L + 32 * j, &mins[j], Laux, -0.9f, 0.05f, 36, 0);
        }
        dblock = make_qp_quants(8, 63, scales, ls, sw);
        mblock = make_qp_quants(8, 63, mins, lm, sw);
        if (five) for (int j = 0; j < 8; ++j) { ls[j] = ls[j] < 63 ? ls[j] : 63; lm[j] = lm[j] < 63 ? lm[j] : 63; }
    }
    pack_scales_k4(y + 4, ls, lm);
    wr16(y, f2h(dblock));
    wr16(y + 2, f2h(mblock));
    for (int j = 0; j < 8; ++j) {
        int sc, m;
        scale_min_k4(j, y + 4, &sc, &m);
        const float d = h2f(rd16(y)) * sc;
        if (!d) continue;
        const float dm = h2f(rd16(y + 2)) * m;
        for (int ii = 0; ii < 32; ++ii) {
            const int l = nearest_int((x[32 * j + ii] + dm) / d);
            L[32 * j + ii] = (uint8_t)IMAX(0, IMIN(nmax, l));
        }
    }
    if (!five) {
        uint8_t *q = y + 16;
        for (int j = 0; j < 256; j += 64, q += 32) for (int l = 0; l < 32; ++l) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
    } else {
        uint8_t *qh = y + 16, *ql = y + 48;
        memset(qh, 0, 32);
        uint8_t m1 = 1, m2 = 2;
        for (int n = 0; n < 256; n += 64, ql += 32, m1 <<= 2, m2 <<= 2)
            for (int j = 0; j < 32; ++j) {
                int l1 = L[n + j], l2 = L[n + j + 32];
                if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
                if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
                ql[j] = (uint8_t)(l1 | (l2 << 4));
            }
    }
}

static void pack_2bit(uint8_t *qs, const uint8_t *L) {
    for (int j = 0; j < 256; j += 128)
        for (int l = 0; l < 32; ++l) qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
}

/* upstream q2_k.cpp:18-106 / :169-242 */
static void quant_q2k_block(const float *x, uint8_t *y, const float *qw) {
    uint8_t L[256], Laux[16], Ls[16], Lm[16];
    float weights[16], mins[16], scales[16], sw[16];
    if (!qw) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 16; ++j) {
            for (int l = 0; l < 16; ++l) weights[l] = fabsf(x[16 * j + l]);
            scales[j] = make_qkx_quants(16, 3, x + 16 * j, weights, L + 16 * j, &mins[j], Laux, -0.5f, 0.1f, 15, 1);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        if (max_scale > 0) {
            const float iscale = 15.f / max_scale;
            for (int j = 0; j < 16; ++j) y[j] = (uint8_t)nearest_int(iscale * scales[j]);
            wr16(y + 80, f2h(max_scale / 15.f));
        } else { memset(y, 0, 16); wr16(y + 80, f2h(0.f)); }
        if (max_min > 0) {
            const float iscale = 15.f / max_min;
            for (int j = 0; j < 16; ++j) y[j] |= (uint8_t)(nearest_int(iscale * mins[j]) << 4);
            wr16(y + 82, f2h(max_min / 15.f));
        } else wr16(y + 82, f2h(0.f));
    } else {
        memset(sw, 0, sizeof sw);
        float sumx2 = 0;
        for (int j = 0; j < 256; ++j) sumx2 += x[j] * x[j];
        const float sigma2 = sumx2 / QK_K;
        for (int j = 0; j < 16; ++j) {
            for (int l = 0; l < 16; ++l) weights[l] = qw[16 * j + l] * sqrtf(sigma2 + x[16 * j + l] * x[16 * j + l]);
            for (int l = 0; l < 16; ++l) sw[j] += weights[l];
            scales[j] = make_qkx_quants(16, 3, x + 16 * j, weights, L + 16 * j, &mins[j], Laux, -0.9f, 0.05f, 36, 0);
        }
        const float dm = make_qp_quants(16, 15, scales, Ls, sw), mm = make_qp_quants(16, 15, mins, Lm, sw);
        wr16(y + 80, f2h(dm));
        wr16(y + 82, f2h(mm));
        for (int j = 0; j < 16; ++j) y[j] = (uint8_t)(Ls[j] | (Lm[j] << 4));
    }
    for (int j = 0; j < 16; ++j) {
        const float d = h2f(rd16(y + 80)) * (y[j] & 0xF);
        if (!d) continue;
        const float dm = h2f(rd16(y + 82)) * (y[j] >> 4);
        for (int ii = 0; ii < 16; ++ii) { const int l = nearest_int((x[16 * j + ii] + dm) / d); L[16 * j + ii] = (uint8_t)IMAX(0, IMIN(3, l)); }
    }
    pack_2bit(y + 16, L);
}

/* upstream q3_k.cpp:18-113 / :176-280 */
static void quant_q3k_block(const float *x, uint8_t *y, const float *qw) {
    int8_t L[256], Ls[16];
    float scales[16], weight[16], sw[16];
    uint8_t *sc_out = y + 96;
    memset(sc_out, 0, 12);
    if (!qw) {
        float max_scale = 0, amax = 0;
        for (int j = 0; j < 16; ++j) {
            scales[j] = make_q3_quants(16, 4, x + 16 * j, L + 16 * j);
            const float a = fabsf(scales[j]);
            if (a > amax) { amax = a; max_scale = scales[j]; }
        }
        if (max_scale) {
            const float iscale = -32.f / max_scale;
            for (int j = 0; j < 16; ++j) {
                int8_t l = (int8_t)nearest_int(iscale * scales[j]);
                l = (int8_t)(IMAX(-32, IMIN(31, l)) + 32);
                Ls[j] = l;
            }
            wr16(y + 108, f2h(1 / iscale));
        } else { memset(Ls, 0, 16); wr16(y + 108, f2h(0.f)); }
    } else {
        float sumx2 = 0;
        for (int j = 0; j < 256; ++j) sumx2 += x[j] * x[j];
        const float sigma2 = 2 * sumx2 / QK_K;
        for (int j = 0; j < 16; ++j) {
            for (int l = 0; l < 16; ++l) weight[l] = qw[16 * j + l] * sqrtf(sigma2 + x[16 * j + l] * x[16 * j + l]);
            float sumw = 0;
            for (int l = 0; l < 16; ++l) sumw += weight[l];
            sw[j] = sumw;
            scales[j] = make_qx_quants(16, 4, x + 16 * j, L + 16 * j, weight);
        }
        const float d_block = make_qx_quants(16, 32, scales, Ls, sw);
        wr16(y + 108, f2h(d_block));
    }
    for (int j = 0; j < 16; ++j) {
        int l = Ls[j];
        if (j < 8) sc_out[j] = (uint8_t)(l & 0xF); else sc_out[j - 8] |= (uint8_t)((l & 0xF) << 4);
        l >>= 4;
        sc_out[j % 4 + 8] |= (uint8_t)(l << (2 * (j / 4)));
    }
    for (int j = 0; j < 16; ++j) {
        int8_t sc = (int8_t)(j < 8 ? sc_out[j] & 0xF : sc_out[j - 8] >> 4);
        sc = (int8_t)((sc | (((sc_out[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32);
        const float d = h2f(rd16(y + 108)) * sc;
        if (!d) continue;
        for (int ii = 0; ii < 16; ++ii) { const int l = nearest_int(x[16 * j + ii] / d); L[16 * j + ii] = (int8_t)(IMAX(-4, IMIN(3, l)) + 4); }
    }
    memset(y, 0, 32);
    int m = 0;
    uint8_t hm = 1;
    for (int j = 0; j < 256; ++j) {
        if (L[j] > 3) { y[m] |= hm; L[j] = (int8_t)(L[j] - 4); }
        if (++m == 32) { m = 0; hm <<= 1; }
    }
    pack_2bit(y + 32, (const uint8_t *)L);
}

/* upstream q6_k.cpp:18-96 / :159-253 */
static void quant_q6k_block(const float *x, uint8_t *y, const float *qw) {
    int8_t L[256];
    float scales[16];
    float max_scale = 0, max_abs_scale = 0;
    for (int ib = 0; ib < 16; ++ib) {
        const float scale = make_qx_quants(16, 32, x + 16 * ib, L + 16 * ib, qw ? qw + 16 * ib : NULL);
        scales[ib] = scale;
        const float a = fabsf(scale);
        if (a > max_abs_scale) { max_abs_scale = a; max_scale = scale; }
    }
    if (max_abs_scale < 1e-15f) { memset(y, 0, 210); wr16(y + 208, f2h(0.f)); return; }
    const float iscale = -128.f / max_scale;
    wr16(y + 208, f2h(1 / iscale));
    int8_t *sc = (int8_t *)(y + 192);
    for (int ib = 0; ib < 16; ++ib) sc[ib] = (int8_t)IMIN(127, nearest_int(iscale * scales[ib]));
    for (int j = 0; j < 16; ++j) {
        const float d = h2f(rd16(y + 208)) * sc[j];
        if (!d) continue;
        for (int ii = 0; ii < 16; ++ii) { const int l = nearest_int(x[16 * j + ii] / d); L[16 * j + ii] = (int8_t)(IMAX(-32, IMIN(31, l)) + 32); }
    }
    uint8_t *ql = y, *qh = y + 128;
    for (int j = 0; j < 256; j += 128, ql += 64, qh += 32)
        for (int l = 0; l < 32; ++l) {
            const uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF, q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
            ql[l] = (uint8_t)(q1 | (q3 << 4));
            ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
            qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
        }
}

/* ------------------------------------------------------------------------------------------- */
/* importance-weighted legacy types: one row.  upstream q4_0.cpp:118-150, q4_1.cpp:59-91,
 * q5_0.cpp:67-107, q5_1.cpp:70-112 */
static void quant_legacy_weighted_row(int type, const float *x, uint8_t *y, int64_t n, const float *qw) {
    float sum_x2 = 0;
    for (int64_t j = 0; j < n; ++j) sum_x2 += x[j] * x[j];
    const float sigma2 = sum_x2 / n;
    const int bytes = type == T_Q4_0 ? 18 : type == T_Q4_1 ? 20 : type == T_Q5_0 ? 22 : 24;
    for (int64_t ib = 0; ib < n / 32; ++ib, y += bytes) {
        const float *xb = x + 32 * ib, *q = qw + 32 * ib;
        float weight[32];
        uint8_t v[32];
        for (int j = 0; j < 32; ++j) weight[j] = q[j] * sqrtf(sigma2 + xb[j] * xb[j]);
        if (type == T_Q4_0 || type == T_Q5_0) {
            int8_t L[32];
            const float d = make_qx_quants(32, type == T_Q4_0 ? 8 : 16, xb, L, weight);
            wr16(y, f2h(d));
            for (int j = 0; j < 32; ++j) v[j] = (uint8_t)L[j];
        } else {
            uint8_t Laux[32];
            float min;
            const float d = make_qkx_quants(32, type == T_Q4_1 ? 15 : 31, xb, weight, v, &min, Laux, -0.9f, 0.05f, 36, 0);
            wr16(y, f2h(d));
            wr16(y + 2, f2h(-min));
        }
        if (type == T_Q4_0) for (int j = 0; j < 16; ++j) y[2 + j] = (uint8_t)(v[j] | (v[j + 16] << 4));
        else if (type == T_Q4_1) for (int j = 0; j < 16; ++j) y[4 + j] = (uint8_t)(v[j] | (v[j + 16] << 4));
        else if (type == T_Q5_0) pack_q5(y + 6, y + 2, v);
        else pack_q5(y + 8, y + 4, v);
    }
}

/* ------------------------------------------------------------------------------------------- */
/* upstream iq4_nl.cpp:13-152 (quantize_row_iq4_nl_impl) with ntry = 7, for one super-block of
 * `sbs` elements (32 for IQ4_NL, 256 for IQ4_XS). */
static void quant_iq4_superblock(int sbs, const float *x, uint8_t *y, const float *qw) {
    const int8_t *values = IQ4NL_VALUES;
    const int nb = sbs / 32;
    uint8_t L[256];
    float scales[8], weight[32];
    float sigma2 = 0;
    for (int j = 0; j < sbs; ++j) sigma2 += x[j] * x[j];
    sigma2 *= 2.f / sbs;
    float max_scale = 0, amax_scale = 0;
    for (int ib = 0; ib < nb; ++ib) {
        const float *xb = x + 32 * ib;
        uint8_t *Lb = L + 32 * ib;
        for (int j = 0; j < 32; ++j) weight[j] = qw ? qw[32 * ib + j] * sqrtf(sigma2 + xb[j] * xb[j]) : xb[j] * xb[j];
        float amax = 0, max = 0;
        for (int j = 0; j < 32; ++j) { const float ax = fabsf(xb[j]); if (ax > amax) { amax = ax; max = xb[j]; } }
        if (amax < 1e-15f) { scales[ib] = 0; memset(Lb, 0, 32); continue; }
        float d = -max / values[0];
        float id = 1 / d;
        float sumqx = 0, sumq2 = 0;
        for (int j = 0; j < 32; ++j) {
            const int l = best_index_int8(values, id * xb[j]);
            Lb[j] = (uint8_t)l;
            const float q = values[l], w = weight[j];
            sumqx += w * q * xb[j];
            sumq2 += w * q * q;
        }
        d = sumq2 > 0 ? sumqx / sumq2 : 0.f;
        float best = d * sumqx;
        for (int itry = -7; itry <= 7; ++itry) {
            id = (itry + values[0]) / max;
            sumqx = sumq2 = 0;
            for (int j = 0; j < 32; ++j) {
                const float q = values[best_index_int8(values, id * xb[j])], w = weight[j];
                sumqx += w * q * xb[j];
                sumq2 += w * q * q;
            }
            if (sumq2 > 0 && sumqx * sumqx > best * sumq2) { d = sumqx / sumq2; best = d * sumqx; }
        }
        scales[ib] = d;
        const float abs_d = fabsf(d);
        if (abs_d > amax_scale) { amax_scale = abs_d; max_scale = d; }
    }
    uint8_t *q4;
    if (nb > 1) {
        uint8_t *scales_l = y + 4;
        uint16_t scales_h = 0;
        q4 = y + 8;
        const float d = -max_scale / 32;
        wr16(y, f2h(d));
        const float id = d ? 1 / d : 0.f;
        for (int ib = 0; ib < nb; ++ib) {
            int l = nearest_int(id * scales[ib]);
            l = IMAX(-32, IMIN(31, l));
            const float dl = d * l, idl = dl ? 1 / dl : 0.f;
            for (int j = 0; j < 32; ++j) L[32 * ib + j] = (uint8_t)best_index_int8(values, idl * x[32 * ib + j]);
            l += 32;
            if (ib % 2 == 0) scales_l[ib / 2] = (uint8_t)(l & 0xf); else scales_l[ib / 2] |= (uint8_t)((l & 0xf) << 4);
            scales_h |= (uint16_t)((l >> 4) << (2 * (ib % 8)));
        }
        wr16(y + 2, scales_h);
    } else {
        q4 = y + 2;
        wr16(y, f2h(scales[0]));
        const float id = scales[0] ? 1 / scales[0] : 0;
        for (int j = 0; j < 32; ++j) L[j] = (uint8_t)best_index_int8(values, id * x[j]);
    }
    for (int i = 0; i < nb; ++i) for (int j = 0; j < 16; ++j) q4[16 * i + j] = (uint8_t)(L[32 * i + j] | (L[32 * i + 16 + j] << 4));
}

/* ------------------------------------------------------------------------------------------- */
/* IQ search tables.  upstream libgguf_iq_tables.cpp:36-417 (iq2xs_init_impl) and :487-666
 * (iq3xs_init_impl): grid coordinates 2*code+1, lattice map, and for every lattice point that is
 * not a codebook entry the codebook entries at the `nwant` smallest distinct squared distances,
 * ordered by (distance, index). */
typedef struct {
    int grid_size, dims, bits;
    uint8_t *grid;      /* grid_size * dims */
    int *map;           /* map_size */
    uint16_t *neighbours;
} iq_table;

static iq_table IQ_TABLES[6]; /* 0 2xxs, 1 2xs, 2 1s, 3 2s, 4 3xxs, 5 3s */

static const iq_table *iq_table_get(int id) {
    iq_table *t = &IQ_TABLES[id];
    if (t->grid) return t;
    static const uint16_t *const books[6] = {CB_IQ2XXS, CB_IQ2XS, CB_IQ1S, CB_IQ2S, CB_IQ3XXS, CB_IQ3S};
    static const int sizes[6] = {256, 512, 2048, 1024, 256, 512};
    static const int nwants[6] = {2, 2, 3, 1, 2, 3};
    const int dims = id < 4 ? 8 : 4, bits = id < 4 ? 2 : 3, map_size = id < 4 ? 43692 : 4096, mask = (1 << bits) - 1;
    const int gs = sizes[id], nwant = nwants[id];
    t->grid_size = gs; t->dims = dims; t->bits = bits;
    uint8_t *grid = (uint8_t *)malloc((size_t)gs * dims);
    int *map = (int *)malloc(sizeof(int) * map_size);
    for (int i = 0; i < map_size; ++i) map[i] = -1;
    for (int g = 0; g < gs; ++g) {
        for (int k = 0; k < dims; ++k) grid[g * dims + k] = (uint8_t)(2 * ((books[id][g] >> (bits * k)) & mask) + 1);
        map[books[id][g]] = g;
    }
    int *d2 = (int *)malloc(sizeof(int) * gs);
    size_t cap = 1 << 16, len = 0;
    uint16_t *nb = (uint16_t *)malloc(cap * sizeof(uint16_t));
    for (int i = 0; i < map_size; ++i) {
        if (map[i] >= 0) continue;
        int pos[8];
        for (int k = 0; k < dims; ++k) pos[k] = 2 * ((i >> (bits * k)) & mask) + 1;
        for (int g = 0; g < gs; ++g) {
            int d = 0;
            for (int k = 0; k < dims; ++k) d += (grid[g * dims + k] - pos[k]) * (grid[g * dims + k] - pos[k]);
            d2[g] = d;
        }
        if (len + (size_t)gs + 1 > cap) { while (len + (size_t)gs + 1 > cap) cap *= 2; nb = (uint16_t *)realloc(nb, cap * sizeof(uint16_t)); }
        map[i] = -((int)len + 1);
        const size_t count_at = len++;
        int have = 0, n = 0, last = -1;
        while (have < nwant) { /* next smallest distinct distance, entries in index order */
            int best = 1 << 30;
            for (int g = 0; g < gs; ++g) if (d2[g] > last && d2[g] < best) best = d2[g];
            if (best == 1 << 30) break;
            for (int g = 0; g < gs; ++g) if (d2[g] == best) { nb[len++] = (uint16_t)g; ++n; }
            last = best;
            ++have;
        }
        nb[count_at] = (uint16_t)n;
    }
    free(d2);
    t->map = map; t->neighbours = nb; t->grid = grid;
    return t;
}

/* upstream libgguf_iq_tables.cpp:434-462 / :683-711 */
static int iq_best_neighbour(const iq_table *t, const uint16_t *nb, const float *xval, const float *weight, float scale, int8_t *L) {
    const int n = nb[0], D = t->dims;
    float best_d2 = 3.402823466e+38f;
    int best = -1;
    for (int j = 1; j <= n; ++j) {
        const uint8_t *pg = t->grid + nb[j] * D;
        float d2 = 0;
        for (int i = 0; i < D; ++i) { const float q = pg[i]; const float diff = scale * q - xval[i]; d2 += weight[i] * diff * diff; }
        if (d2 < best_d2) { best_d2 = d2; best = nb[j]; }
    }
    const uint8_t *pg = t->grid + best * D;
    for (int i = 0; i < D; ++i) L[i] = (int8_t)((pg[i] - 1) / 2);
    return best;
}

/* upstream libgguf_iq_tables.cpp:714-781 (reachable part) */
static int iq1_best_neighbour(const iq_table *t, const uint16_t *nb, const float *xval, const float *weight, float scale,
                              const float *xg, int8_t *L) {
    const int n = nb[0];
    float best_score = 3.402823466e+38f;
    int best = -1;
    for (int j = 1; j <= n; ++j) {
        const uint8_t *pg = t->grid + nb[j] * 8;
        float d2 = 0;
        for (int i = 0; i < 8; ++i) { const float q = xg[(pg[i] - 1) / 2]; const float diff = scale * q - xval[i]; d2 += weight[i] * diff * diff; }
        if (d2 < best_score) { best_score = d2; best = nb[j]; }
    }
    const uint8_t *pg = t->grid + best * 8;
    for (int i = 0; i < 8; ++i) L[i] = (int8_t)((pg[i] - 1) / 2);
    return best;
}

/* One super-block of IQ2_XXS / IQ2_XS / IQ2_S / IQ3_XXS / IQ3_S.
 * upstream iq2_xxs.cpp:4-224, iq2_xs.cpp:4-230, iq2_s.cpp:4-218, iq3_xxs.cpp:4-273, iq3_s.cpp:5-233. */
static void quant_iq23_block(int type, const float *xbl, uint8_t *y, const float *qw_block) {
    const int xxs2 = type == T_IQ2_XXS, xs2 = type == T_IQ2_XS, s2 = type == T_IQ2_S, xxs3 = type == T_IQ3_XXS, s3 = type == T_IQ3_S;
    const int BS = (xs2 || s2) ? 16 : 32, GD = (xxs3 || s3) ? 4 : 8, BITS = GD == 8 ? 2 : 3, KMAXQ = GD == 8 ? 3 : 8;
    const int NG = BS / GD, NS = BS / 8, NB = 256 / BS;
    const int parity = xxs2 || xs2 || xxs3;
    const int is_max = xxs2 ? 6 : xxs3 ? 15 : 9;
    const float step = GD == 8 ? 0.1f : 0.2f;
    const iq_table *t = iq_table_get(xxs2 ? 0 : xs2 ? 1 : s2 ? 3 : xxs3 ? 4 : 5);
    int bytes, e_;
    block_geometry(type, &e_, &bytes);
    memset(y, 0, (size_t)bytes);
    float scales[16];
    float sumx2 = 0;
    for (int i = 0; i < 256; ++i) sumx2 += xbl[i] * xbl[i];
    const float sigma2 = (xxs2 || xs2) ? sumx2 / QK_K : 2 * sumx2 / QK_K;
    float max_scale = 0;
    int pos = 0; /* IQ3_S: payload slot, advanced only by blocks that are not skipped */
    for (int ib = 0; ib < NB; ++ib) {
        const float *xb = xbl + BS * ib;
        float weight[32], waux[32], xval[32];
        int8_t L[32], Laux[32];
        uint8_t signs[4];
        for (int i = 0; i < BS; ++i) {
            if (qw_block) weight[i] = qw_block[BS * ib + i] * sqrtf(sigma2 + xb[i] * xb[i]);
            else weight[i] = s2 ? 0.25f * sigma2 + xb[i] * xb[i] : xb[i] * xb[i];
        }
        for (int i = 0; i < BS; ++i) waux[i] = sqrtf(weight[i]);
        for (int k = 0; k < NS; ++k) {
            int nflip = 0;
            uint8_t s = 0;
            for (int i = 0; i < 8; ++i) {
                if (xb[8 * k + i] >= 0) xval[8 * k + i] = xb[8 * k + i];
                else { xval[8 * k + i] = -xb[8 * k + i]; ++nflip; s |= (uint8_t)(1 << i); }
            }
            if (parity) {
                if (nflip % 2) {
                    int imin = 0;
                    float min = weight[8 * k] * xb[8 * k] * xb[8 * k];
                    for (int i = 1; i < 8; ++i) { const float ax = weight[8 * k + i] * xb[8 * k + i] * xb[8 * k + i]; if (ax < min) { min = ax; imin = i; } }
                    xval[8 * k + imin] = -xval[8 * k + imin];
                    s ^= (uint8_t)(1 << imin);
                }
                s &= 127;
            }
            signs[k] = s;
        }
        float max = xval[0];
        for (int i = 1; i < BS; ++i) max = max > xval[i] ? max : xval[i];
        memset(L, 0, sizeof L);
        int skipped = s3 ? !max : (max < ((s2 || xxs3) ? 1e-8f : 1e-15f));
        float scale = 0, eff_max = max;
        if (!skipped && xxs2) {
            scale = make_qp_quants(32, KMAXQ + 1, xval, (uint8_t *)L, weight);
            eff_max = scale * KMAXQ;
            if (eff_max <= 0) { skipped = 1; memset(L, 0, sizeof L); }
        }
        if (skipped) { scales[ib] = 0; continue; }
        float best = 0;
        if (!xxs2) scale = max / (2 * KMAXQ - 1);
        int on_grid[8], on_aux[8];
        for (int k = 0; k < NG; ++k) on_grid[k] = !s3;
        for (int is = -is_max; is <= is_max; ++is) {
            const float id = (2 * KMAXQ - 1 + is * step) / eff_max;
            const float this_scale = 1 / id;
            for (int k = 0; k < NG; ++k) {
                uint16_t u = 0;
                for (int i = 0; i < GD; ++i) {
                    const int l = nearest_int(0.5f * (id * xval[GD * k + i] - 1));
                    Laux[GD * k + i] = (int8_t)IMAX(0, IMIN(KMAXQ - 1, l));
                    u |= (uint16_t)(Laux[GD * k + i] << (BITS * i));
                }
                on_aux[k] = 1;
                if (t->map[u] < 0) {
                    on_aux[k] = 0;
                    iq_best_neighbour(t, t->neighbours - t->map[u] - 1, xval + GD * k, waux + GD * k, this_scale, Laux + GD * k);
                }
            }
            float sumqx = 0, sumq2 = 0;
            for (int i = 0; i < BS; ++i) { const float w = weight[i], q = 2 * Laux[i] + 1; sumqx += w * xval[i] * q; sumq2 += w * q * q; }
            if (sumq2 > 0 && sumqx * sumqx > best * sumq2) {
                scale = sumqx / sumq2; best = scale * sumqx;
                memcpy(L, Laux, (size_t)BS);
                for (int k = 0; k < NG; ++k) on_grid[k] = on_aux[k];
            }
        }
        int n_not = 0;
        for (int k = 0; k < NG; ++k) if (!on_grid[k]) ++n_not;
        if ((xxs2 ? 1 : n_not > 0) && scale > 0) {
            const float id = 1 / scale;
            for (int k = 0; k < NG; ++k) {
                if (!(xxs2 || s3) && on_grid[k]) continue;
                uint16_t u = 0;
                int8_t Lr[8];
                for (int i = 0; i < GD; ++i) {
                    const int l = IMAX(0, IMIN(KMAXQ - 1, nearest_int(0.5f * (id * xval[GD * k + i] - 1))));
                    u |= (uint16_t)(l << (BITS * i));
                    Lr[i] = (int8_t)l;
                }
                int g = t->map[u];
                if (xs2 || s2) {
                    if (g < 0) iq_best_neighbour(t, t->neighbours - g - 1, xval + GD * k, waux + GD * k, scale, Lr);
                    memcpy(L + GD * k, Lr, (size_t)GD);
                } else {
                    if (g < 0) g = iq_best_neighbour(t, t->neighbours - g - 1, xval + GD * k, waux + GD * k, scale, Lr);
                    for (int i = 0; i < GD; ++i) L[GD * k + i] = (int8_t)((t->grid[g * GD + i] - 1) / 2);
                }
            }
            float sumqx = 0, sumq2 = 0;
            for (int i = 0; i < BS; ++i) { const float w = weight[i], q = 2 * L[i] + 1; sumqx += w * xval[i] * q; sumq2 += w * q * q; }
            if (sumq2 > 0) scale = sumqx / sumq2;
        }
        if (scale < 0) {
            scale = -scale;
            for (int k = 0; k < NS; ++k) signs[k] = (uint8_t)(parity ? (~signs[k]) & 127 : ~signs[k]);
        }
        int gi[8];
        for (int k = 0; k < NG; ++k) {
            uint16_t u = 0;
            for (int i = 0; i < GD; ++i) u |= (uint16_t)(L[GD * k + i] << (BITS * i));
            gi[k] = t->map[u] < 0 ? 0 : t->map[u];
        }
        if (xxs2) {
            uint32_t w0 = 0, w1 = 0;
            for (int k = 0; k < 4; ++k) { w0 |= (uint32_t)gi[k] << (8 * k); w1 |= (uint32_t)signs[k] << (7 * k); }
            wr32(y + 2 + 8 * ib, w0);
            wr32(y + 2 + 8 * ib + 4, w1);
        } else if (xs2) {
            for (int k = 0; k < 2; ++k) wr16(y + 2 + 2 * (2 * ib + k), (uint16_t)(gi[k] | (signs[k] << 9)));
        } else if (s2) {
            for (int k = 0; k < 2; ++k) {
                const int i8 = 2 * ib + k;
                y[2 + i8] = (uint8_t)(gi[k] & 255);
                y[66 + i8 / 4] |= (uint8_t)((gi[k] >> 8) << (2 * (i8 % 4)));
                y[2 + 32 + i8] = signs[k];
            }
        } else if (xxs3) {
            for (int k = 0; k < 8; ++k) y[2 + 8 * ib + k] = (uint8_t)gi[k];
            wr32(y + 66 + 4 * ib, (uint32_t)signs[0] | ((uint32_t)signs[1] << 7) | ((uint32_t)signs[2] << 14) | ((uint32_t)signs[3] << 21));
        } else {
            for (int k = 0; k < 8; ++k) {
                y[2 + 8 * pos + k] = (uint8_t)(gi[k] & 255);
                y[66 + ib] |= (uint8_t)((gi[k] >> 8) << k);
            }
            for (int k = 0; k < 4; ++k) y[74 + 4 * pos + k] = signs[k];
            ++pos;
        }
        scales[ib] = scale;
        max_scale = max_scale > scale ? max_scale : scale;
    }
    if (!max_scale) {
        if (xxs2 || xs2 || xxs3) memset(y, 0, (size_t)bytes);
        return;
    }
    const float d = max_scale / 31;
    wr16(y, f2h(s2 ? d * 0.9875f : xxs3 ? d * 1.0125f : s3 ? d * 1.033f : d));
    const float id = 1 / d;
    for (int ib = 0; ib < NB; ++ib) {
        const int l = IMAX(0, IMIN(15, nearest_int(0.5f * (id * scales[ib] - 1))));
        if (xxs2) { const uint32_t w1 = rd32(y + 2 + 8 * ib + 4) | ((uint32_t)l << 28); wr32(y + 2 + 8 * ib + 4, w1); }
        else if (xxs3) { const uint32_t w = rd32(y + 66 + 4 * ib) | ((uint32_t)l << 28); wr32(y + 66 + 4 * ib, w); }
        else {
            uint8_t *sc = y + (xs2 ? 66 : s2 ? 74 : 106) + ib / 2;
            if (ib % 2 == 0) *sc = (uint8_t)l; else *sc |= (uint8_t)(l << 4);
        }
    }
}

static int cmp_pair_value(const void *a, const void *b) {
    const float l = *(const float *)a, r = *(const float *)b;
    return l < r ? -1 : l > r ? 1 : 0;
}

/* One super-block of IQ1_S (32-element blocks) or IQ1_M (16-element blocks).
 * upstream iq1_s.cpp:6-204, iq1_m.cpp:4-318.  The sort must keep equal values in index order
 * (what upstream's qsort does in the C library it is built against); an insertion sort is used. */
static void quant_iq1_block(int is_m, const float *xbl, uint8_t *y, const float *qw_block) {
    const int BS = is_m ? 16 : 32, NB = 256 / BS, NG = BS / 8;
    const iq_table *t = iq_table_get(2);
    const float x_p[3] = {-1 + 0.125f, 0.125f, 1 + 0.125f}, x_m[3] = {-1 - 0.125f, -0.125f, 1 - 0.125f};
    static const uint8_t masks[4] = {0x00, 0x80, 0x08, 0x88};
    memset(y, 0, is_m ? 56 : 50);
    float scales[16];
    int shifts[16];
    float sumx2 = 0;
    for (int i = 0; i < 256; ++i) sumx2 += xbl[i] * xbl[i];
    const float sigma2 = 2 * sumx2 / QK_K;
    float max_scale = 0;
    (void)cmp_pair_value;
    for (int ib = 0; ib < NB; ++ib) {
        const float *xb = xbl + BS * ib;
        float weight[32];
        int8_t L[32];
        for (int i = 0; i < BS; ++i) weight[i] = qw_block ? qw_block[BS * ib + i] * sqrtf(sigma2 + xb[i] * xb[i]) : xb[i] * xb[i];
        float max = fabsf(xb[0]);
        for (int i = 1; i < BS; ++i) max = max > fabsf(xb[i]) ? max : fabsf(xb[i]);
        scales[ib] = 0;
        shifts[ib] = is_m ? 0 : 1;
        if (max < (is_m ? 1e-7f : 1e-12f)) continue;
        int idx[32];
        float val[32];
        for (int j = 0; j < BS; ++j) {
            const float v = xb[j];
            int p = j - 1;
            while (p >= 0 && val[p] > v) { val[p + 1] = val[p]; idx[p + 1] = idx[p]; --p; }
            val[p + 1] = v; idx[p + 1] = j;
        }
        float best_score = -3.402823466e+38f, scale = max;
        int besti1 = -1, besti2 = -1, best_k = is_m ? -1 : 0;
        if (!is_m) {
            float sumx[33], sumw[33];
            sumx[0] = sumw[0] = 0;
            for (int j = 0; j < BS; ++j) { const int i = idx[j]; sumx[j + 1] = sumx[j] + weight[i] * xb[i]; sumw[j + 1] = sumw[j] + weight[i]; }
            for (int i1 = 0; i1 <= BS; ++i1)
                for (int i2 = i1; i2 <= BS; ++i2) {
                    float sumqx = (sumx[i1] - sumx[0]) * x_p[0] + (sumx[i2] - sumx[i1]) * x_p[1] + (sumx[BS] - sumx[i2]) * x_p[2];
                    float sumq2 = (sumw[i1] - sumw[0]) * x_p[0] * x_p[0] + (sumw[i2] - sumw[i1]) * x_p[1] * x_p[1] + (sumw[BS] - sumw[i2]) * x_p[2] * x_p[2];
                    if (sumq2 > 0 && sumqx * sumqx > best_score * sumq2) { scale = sumqx / sumq2; best_score = scale * sumqx; besti1 = i1; besti2 = i2; best_k = 1; }
                    sumqx = (sumx[i1] - sumx[0]) * x_m[0] + (sumx[i2] - sumx[i1]) * x_m[1] + (sumx[BS] - sumx[i2]) * x_m[2];
                    sumq2 = (sumw[i1] - sumw[0]) * x_m[0] * x_m[0] + (sumw[i2] - sumw[i1]) * x_m[1] * x_m[1] + (sumw[BS] - sumw[i2]) * x_m[2] * x_m[2];
                    if (sumq2 > 0 && sumqx * sumqx > best_score * sumq2) { scale = sumqx / sumq2; best_score = scale * sumqx; besti1 = i1; besti2 = i2; best_k = -1; }
                }
            if (besti1 < 0 || besti2 < 0 || best_k == 0) continue;
        } else {
            for (int i1 = 0; i1 <= BS; ++i1)
                for (int i2 = i1; i2 <= BS; ++i2) {
                    float sqx[4] = {0, 0, 0, 0}, sq2[4] = {0, 0, 0, 0};
                    for (int j = 0; j < BS; ++j) {
                        const int i = idx[j], lv = j < i1 ? 0 : (j < i2 ? 1 : 2), lo = i < BS / 2;
                        const float ap = weight[i] * x_p[lv] * xb[i], am = weight[i] * x_m[lv] * xb[i];
                        const float bp = weight[i] * x_p[lv] * x_p[lv], bm = weight[i] * x_m[lv] * x_m[lv];
                        sqx[0] += ap; sqx[1] += lo ? ap : am; sqx[2] += lo ? am : ap; sqx[3] += am;
                        sq2[0] += bp; sq2[1] += lo ? bp : bm; sq2[2] += lo ? bm : bp; sq2[3] += bm;
                    }
                    for (int k = 0; k < 4; ++k)
                        if (sq2[k] > 0 && sqx[k] * sqx[k] > best_score * sq2[k]) { scale = sqx[k] / sq2[k]; best_score = scale * sqx[k]; besti1 = i1; besti2 = i2; best_k = k; }
                }
            if (besti1 < 0 || besti2 < 0 || best_k < 0) continue;
        }
        for (int j = 0; j < BS; ++j) L[idx[j]] = (int8_t)(j < besti1 ? 0 : (j < besti2 ? 1 : 2));
        if (scale < 0) {
            for (int j = 0; j < BS; ++j) L[j] = (int8_t)(2 - L[j]);
            scale = -scale;
            best_k = is_m ? 3 - best_k : -best_k;
        }
        int all_on_grid = 1, index[4];
        for (int k = 0; k < NG; ++k) {
            const int plus = is_m ? (k == 0 ? best_k < 2 : best_k % 2 == 0) : best_k == 1;
            const float *xx = plus ? x_p : x_m;
            uint16_t u = 0;
            for (int j = 0; j < 8; ++j) u |= (uint16_t)(L[8 * k + j] << (2 * j));
            int g = t->map[u];
            if (g < 0) { all_on_grid = 0; g = iq1_best_neighbour(t, t->neighbours - g - 1, xb + 8 * k, weight + 8 * k, scale, xx, L + 8 * k); }
            index[k] = g;
        }
        if (!all_on_grid) {
            float sumqx = 0, sumq2 = 0;
            for (int k = 0; k < NG; ++k) {
                const int plus = is_m ? (k == 0 ? best_k < 2 : best_k % 2 == 0) : best_k == 1;
                const float *xx = plus ? x_p : x_m;
                const uint8_t *pg = t->grid + index[k] * 8;
                for (int j = 0; j < 8; ++j) { const float w = weight[8 * k + j], q = xx[(pg[j] - 1) / 2]; sumqx += w * q * xb[8 * k + j]; sumq2 += w * q * q; }
            }
            if (sumqx > 0 && sumq2 > 0) scale = sumqx / sumq2;
        }
        if (!is_m) {
            uint16_t h = 0;
            for (int k = 0; k < 4; ++k) { y[2 + 4 * ib + k] = (uint8_t)(index[k] & 255); h |= (uint16_t)((index[k] >> 8) << (3 * k)); }
            wr16(y + 34 + 2 * ib, h);
        } else {
            y[2 * ib] = (uint8_t)(index[0] & 255);
            y[2 * ib + 1] = (uint8_t)(index[1] & 255);
            y[32 + ib] = (uint8_t)((index[0] >> 8) | ((index[1] >> 8) << 4));
        }
        scales[ib] = scale;
        shifts[ib] = best_k;
        max_scale = max_scale > scale ? max_scale : scale;
    }
    if (!max_scale) return;
    float d = max_scale / 15;
    const float id = 1 / d;
    if (!is_m) {
        wr16(y, f2h(d * 1.125f));
        for (int ib = 0; ib < NB; ++ib) {
            int l = IMAX(0, IMIN(7, nearest_int(0.5f * (id * scales[ib] - 1))));
            if (shifts[ib] == -1) l |= 8;
            wr16(y + 34 + 2 * ib, (uint16_t)(rd16(y + 34 + 2 * ib) | (l << 12)));
        }
        return;
    }
    uint16_t sc[4] = {0, 0, 0, 0};
    float sumqx_f = 0, sumq2_f = 0;
    for (int ib = 0; ib < NB; ++ib) {
        const int l = IMAX(0, IMIN(7, nearest_int(0.5f * (id * scales[ib] - 1))));
        sc[ib / 4] |= (uint16_t)(l << (3 * (ib % 4)));
        y[32 + ib] |= masks[shifts[ib]];
        const float *xb = xbl + BS * ib;
        for (int k = 0; k < 2; ++k) {
            const int plus = k == 0 ? shifts[ib] < 2 : shifts[ib] % 2 == 0;
            const float *xx = plus ? x_p : x_m;
            const uint8_t *pg = t->grid + 8 * (y[2 * ib + k] + ((y[32 + ib] << (8 - 4 * k)) & 0x700));
            for (int j = 0; j < 8; ++j) {
                const float w = qw_block ? qw_block[BS * ib + 8 * k + j] * sqrtf(sigma2 + xb[8 * k + j] * xb[8 * k + j]) : xb[8 * k + j] * xb[8 * k + j];
                const float q = xx[(pg[j] - 1) / 2] * (2 * l + 1);
                sumqx_f += w * q * xb[8 * k + j];
                sumq2_f += w * q * q;
            }
        }
    }
    if (sumq2_f > 0) d = sumqx_f / sumq2_f;
    const uint16_t s = f2h(d * 1.1125f);
    sc[0] |= (uint16_t)((s & 0x000f) << 12);
    sc[1] |= (uint16_t)((s & 0x00f0) << 8);
    sc[2] |= (uint16_t)((s & 0x0f00) << 4);
    sc[3] |= (uint16_t)(s & 0xf000);
    for (int k = 0; k < 4; ++k) wr16(y + 48 + 2 * k, sc[k]);
}

/* ------------------------------------------------------------------------------------------- */
int gguf_oracle_quantize_supported(int type) {
    switch (type) {
        case T_F32: case T_F16: case T_BF16:
        case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_Q8_0: case T_Q1_0: case T_MXFP4: case T_NVFP4:
        case T_TQ1_0: case T_TQ2_0: case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K:
        case T_IQ4_NL: case T_IQ4_XS:
        case T_IQ2_XXS: case T_IQ2_XS: case T_IQ2_S: case T_IQ3_XXS: case T_IQ3_S: case T_IQ1_S: case T_IQ1_M:
            return 1;
        default:
            return 0;
    }
}

/* upstream libgguf.cpp:311-405 (serial chunk) */
size_t gguf_oracle_quantize_chunk(int type, const float *src, void *dst, int64_t start, int64_t nrows, int64_t n,
                                  const float *imatrix) {
    if (nrows <= 0) return 0;
    const size_t rs = gguf_oracle_row_size(type, n);
    if (rs == 0 || start < 0 || start % n != 0 || !gguf_oracle_quantize_supported(type)) return 0;
    if (gguf_oracle_quantize_requires_imatrix(type) && !imatrix) return 0;
    const float *x = src + start;
    uint8_t *y = (uint8_t *)dst + (size_t)(start / n) * rs;
    const int64_t k = nrows * n;
    switch (type) {
        case T_F32: memcpy(y, x, (size_t)k * 4); return (size_t)k * 4;
        case T_F16: for (int64_t i = 0; i < k; ++i) wr16(y + 2 * i, f2h(x[i])); return (size_t)k * 2;
        case T_BF16: for (int64_t i = 0; i < k; ++i) wr16(y + 2 * i, f2bf(x[i])); return (size_t)k * 2;
        case T_Q8_0: quant_q8_0(x, y, k); break;
        case T_Q1_0: quant_q1_0(x, y, k); break;
        case T_MXFP4: quant_mxfp4(x, y, k); break;
        case T_NVFP4: quant_nvfp4(x, y, k); break;
        case T_TQ1_0: quant_ternary(x, y, k, 1); break;
        case T_TQ2_0: quant_ternary(x, y, k, 0); break;
        case T_Q4_0: case T_Q5_0: case T_Q4_1: case T_Q5_1:
            if (imatrix) {
                for (int64_t r = 0; r < nrows; ++r) quant_legacy_weighted_row(type, x + r * n, y + r * rs, n, imatrix);
            } else if (type == T_Q4_0 || type == T_Q5_0) quant_q4_0_q5_0(x, y, k, type == T_Q5_0);
            else quant_q4_1_q5_1(x, y, k, type == T_Q5_1);
            break;
        case T_IQ2_XXS: case T_IQ2_XS: case T_IQ2_S: case T_IQ3_XXS: case T_IQ3_S: case T_IQ1_S: case T_IQ1_M:
        case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K: case T_IQ4_XS: case T_IQ4_NL: {
            int e, b;
            block_geometry(type, &e, &b);
            const int64_t per_row = n / e;
            for (int64_t r = 0; r < nrows; ++r)
                for (int64_t i = 0; i < per_row; ++i) {
                    const float *xb = x + r * n + i * e;
                    uint8_t *yb = y + r * rs + i * b;
                    const float *qw = imatrix ? imatrix + i * e : NULL;
                    if (type == T_Q2_K) quant_q2k_block(xb, yb, qw);
                    else if (type == T_Q3_K) quant_q3k_block(xb, yb, qw);
                    else if (type == T_Q6_K) quant_q6k_block(xb, yb, qw);
                    else if (type == T_IQ4_XS) quant_iq4_superblock(256, xb, yb, qw);
                    else if (type == T_IQ4_NL) quant_iq4_superblock(32, xb, yb, qw);
                    else if (type == T_IQ1_S || type == T_IQ1_M) quant_iq1_block(type == T_IQ1_M, xb, yb, qw);
                    else if (type == T_IQ2_XXS || type == T_IQ2_XS || type == T_IQ2_S || type == T_IQ3_XXS || type == T_IQ3_S) quant_iq23_block(type, xb, yb, qw);
                    else quant_q4k_q5k_block(xb, yb, qw, type == T_Q5_K);
                }
        } break;
        default: return 0;
    }
    return (size_t)nrows * rs;
}
