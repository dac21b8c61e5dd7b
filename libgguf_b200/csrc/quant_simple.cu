// Memory-bound quantizers: Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q1_0, MXFP4, NVFP4, TQ1_0, TQ2_0
// (the paths taken when no importance weights are given; the weighted legacy variants live
// with the K-quant search code).
//
// 32-element types: a CTA stages 128 runs of 32 floats in shared memory with coalesced 16-byte
// loads, then every thread encodes one run from registers, serially and in upstream's element
// order, and the encoded tile is written out as 16-byte vectors.  The encoders are written to
// keep the instruction count per element low (the kernels are issue-bound long before they are
// memory-bound): rounding by directed-rounding adds of 2^23 instead of conversions, FP4 levels
// by the hardware E2M1 conversion wrapped so that it reproduces upstream's scan exactly.
#include <float.h>
#include <math.h>

#include "bulk_copy.cuh"
#include "gguf_common.cuh"
#include "gguf_tables.cuh"
#include "kernels.h"
#include "tile_io.cuh"

namespace gguf {
namespace {

constexpr int kThreads = 256;
constexpr unsigned kFull = 0xffffffffu;
constexpr float kInfinity = __builtin_huge_valf();

// The 16-way nearest-level scan of the FP4 formats (upstream libgguf_common.h:321-335):
// first index with the smallest |level*e - x|.
GGUF_D int best_index_fp4_scan(float x, float e) {
    int best = 0;
    float best_err = fabsf((float)k_fp4_values[0] * e - x);
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        const float err = fabsf((float)k_fp4_values[i] * e - x);
        if (err < best_err) { best = i; best_err = err; }
    }
    return best;
}

// Same result as the scan, by thresholds.  The levels are +-{0,1,2,3,4,6,8,12}*e; level*e is exact
// (e has at most 4 significant bits), and for the two levels adjacent to |x| the differences the
// scan compares are exact too (Sterbenz), so the scan's winner is the true nearest magnitude with
// ties going to the smaller one (it comes first in scan order, for both signs), i.e. the number
// of midpoints {0.5,1.5,2.5,3.5,5,7,10}*e strictly below |x|.  Farther levels cannot tie with the
// nearest while |x| < 2^20*e (their distance exceeds the nearest's by at least e, far above the
// rounding of the subtraction); beyond that, for e == 0 and for NaN the scan itself is used.
// Checked against the scan over all 2^32 inputs for a set of scales by libgguf_cuda_selftest_fp4.
GGUF_D bool fp4_thresholds_valid(float amax, float e) { return amax <= e * 1048576.f && e != 0.f; }  // false for NaN too
GGUF_D int best_index_fp4_thresholds(float x, float e) {
    const float m = fabsf(x);
    int idx = (m > 0.5f * e) + (m > 1.5f * e) + (m > 2.5f * e) + (m > 3.5f * e) + (m > 5.f * e) + (m > 7.f * e) + (m > 10.f * e);
    if (x < 0.f && idx > 0) idx += 8;
    return idx;
}
GGUF_D int best_index_fp4(float x, float e) {
    return fp4_thresholds_valid(fabsf(x), e) ? best_index_fp4_thresholds(x, e) : best_index_fp4_scan(x, e);
}

// ---- FP4 levels by the hardware conversion ----------------------------------------------------
// cvt.rn.satfinite.e2m1x2.f32 rounds to the nearest E2M1 value {0,.5,1,1.5,2,3,4,6} (saturating),
// ties to even; upstream's scan picks the nearest of {0,1,2,3,4,6,8,12}*e with ties to the smaller
// magnitude, and never emits the code of -0.  The two agree wherever the scaled input is not an
// exact tie, so the wrappers below keep exact ties away from the instruction.
//
// Four bytes of codes: byte k = code(hi[k]) << 4 | code(lo[k]).
GGUF_D uint32_t cvt_e2m1x8(const float *lo, const float *hi) {
    uint32_t r;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %1, %2;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %3, %4;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %5, %6;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %7, %8;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}"
        : "=r"(r)
        : "f"(hi[0]), "f"(lo[0]), "f"(hi[1]), "f"(lo[1]), "f"(hi[2]), "f"(lo[2]), "f"(hi[3]), "f"(lo[3]));
    return r;
}
// Code 8 (-0) -> 0 in each of the eight nibbles: the scan returns the first best index, which is 0.
GGUF_D uint32_t drop_negative_zero(uint32_t w) {
    const uint32_t mag = w & 0x77777777u;
    const uint32_t nonzero = (mag + 0x77777777u) & 0x88888888u;  // bit 3 of a nibble set iff its magnitude is not 0
    return mag | (w & nonzero);
}

// Power-of-two scale (MXFP4), e = 2^(ebyte-128) being the value of level 1.  x * 2^(127-ebyte) is
// exact, and multiplying by (1 - 2^-24) with rounding toward zero steps a float to its predecessor
// in magnitude; "predecessor | 1" is x itself when x's last mantissa bit is 1 and the predecessor
// when it is 0.  Every tie has a zero last bit, so ties move just below themselves (-> smaller
// magnitude, as the scan does) and no other value crosses a tie.
// scale_rz = 2^(127-ebyte) * (1 - 2^-24), exactly representable for ebyte <= 252.
GGUF_D float mx_scale_rz(int ebyte) { return __uint_as_float(((uint32_t)(254 - ebyte) << 23) - 1u); }
GGUF_D float mx_nudge(float x, float scale_rz) { return __uint_as_float(__float_as_uint(__fmul_rz(x, scale_rz)) | 1u); }

// Any scale (NVFP4): the quotient x / (2e) is bracketed by two products that lie strictly on either
// side of it (relative distance 2^-21, far above the error of the approximate reciprocal, about 2^-23,
// and of the product).  The
// scan's answer is monotone in the quotient and equals the conversion away from ties, so where both
// ends convert to the same code that code is the answer; where they differ (a tie lies between the
// ends, in practice: the input is a tie) the element is redone by the exact search.
struct Fp4Bracket { float lo, hi; };
GGUF_D Fp4Bracket fp4_bracket(float e) {
    float inv;
    asm("rcp.approx.f32 %0, %1;" : "=f"(inv) : "f"(e + e));  // e >= 2^-10: no denormal in or out
    return {inv * 0.99999952316284179688f, inv * 1.00000047683715820312f};  // 1 -+ 2^-21
}
// bit 4n set when nibble n of v is not zero
GGUF_D uint32_t nonzero_nibbles(uint32_t v) {
    v |= v >> 1;
    v |= v >> 2;
    return v & 0x11111111u;
}
// Codes of elements x[0..3] (low nibbles) and y[0..3] (high nibbles) of four bytes by the lower end of the
// bracket; `other` gets the nibbles (XOR) by which the upper end's codes differ: non-zero exactly where a tie
// lies between the two ends.
GGUF_D uint32_t fp4_word_bracketed(const float *x, const float *y, const Fp4Bracket &k, uint32_t &other) {
    float lo_a[4], hi_a[4], lo_b[4], hi_b[4];
    const float2 klo = make_float2(k.lo, k.lo), khi = make_float2(k.hi, k.hi);
#pragma unroll
    for (int i = 0; i < 4; i += 2) {  // two neighbouring elements per multiply instruction (nothing is added to the products)
        const float2 xx = make_float2(x[i], x[i + 1]), yy = make_float2(y[i], y[i + 1]);
        const float2 a = __fmul2_rn(xx, klo), b = __fmul2_rn(yy, klo), c = __fmul2_rn(xx, khi), d = __fmul2_rn(yy, khi);
        lo_a[i] = a.x; lo_a[i + 1] = a.y;
        hi_a[i] = b.x; hi_a[i + 1] = b.y;
        lo_b[i] = c.x; lo_b[i + 1] = c.y;
        hi_b[i] = d.x; hi_b[i + 1] = d.y;
    }
    const uint32_t a = drop_negative_zero(cvt_e2m1x8(lo_a, hi_a)), b = drop_negative_zero(cvt_e2m1x8(lo_b, hi_b));
    other = a ^ b;
    return a;
}
// Settles the nibbles of `word` that the bracket left open.  The two candidate codes are neighbours; the scan
// takes the larger magnitude only when |x| lies strictly above their midpoint {0.5,1.5,2.5,3.5,5,7,10}[m] * e
// (m = the smaller code's magnitude bits; the product is exact).  x: the sub-block in shared memory; nibble n
// of word w is element 4w + n/2 (low halves) or 8 + 4w + n/2 (high halves).
GGUF_D uint32_t fp4_settle(uint32_t word, uint32_t other, const float *x, int w, float e) {
    uint32_t open = nonzero_nibbles(other);
    const float half_e = 0.5f * e;
    while (open) {
        const int bit = __ffs((int)open) - 1;  // 4n
        open &= open - 1;
        const uint32_t m = (word >> bit) & 7u;
        const uint32_t twice_mid = (0x140E0A07050301ull >> (8 * m)) & 0xFFu;
        const float v = x[4 * w + (bit >> 3) + ((bit & 4) ? 8 : 0)];
        if (fabsf(v) > (float)twice_mid * half_e) word ^= other & (0xFu << bit);
    }
    return word;
}
// mode 0: threshold search against the scan.  mode 1: power-of-two-scale hardware path (e is
// 2^(ebyte-128), ebyte <= 252).  mode 2: bracketed hardware path; inputs whose bracket straddles a
// tie are settled by the midpoint comparison and counted in `fallbacks`.  Modes 1 and 2 only look
// at the inputs the quantizers send down those paths (|x| <= 2^20 * e).
__global__ void selftest_fp4_kernel(float e, int mode, int ebyte, unsigned long long *mismatches, unsigned long long *fallbacks) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    unsigned long long bad = 0, fell = 0;
    const float scale_rz = mx_scale_rz(ebyte);
    for (uint64_t bits = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; bits < (1ull << 32); bits += stride) {
        const float x = __uint_as_float((uint32_t)bits);
        const int want = best_index_fp4_scan(x, e);
        if (mode == 0) {
            if (best_index_fp4(x, e) != want) ++bad;
            continue;
        }
        if (!(fabsf(x) < kInfinity) || !fp4_thresholds_valid(fabsf(x), e)) continue;
        float lo[4] = {x, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
        if (mode == 1) {
            lo[0] = mx_nudge(x, scale_rz);
            if ((int)(drop_negative_zero(cvt_e2m1x8(lo, hi)) & 0xFu) != want) ++bad;
        } else {
            float xs[8] = {x, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            uint32_t other;
            uint32_t word = fp4_word_bracketed(xs, xs + 4, fp4_bracket(e), other);
            if (other & 0xFu) {
                ++fell;
                word = fp4_settle(word, other & 0xFu, xs, 0, e);
            }
            if ((int)(word & 0xFu) != want) ++bad;
        }
    }
    if (bad) atomicAdd(mismatches, bad);
    if (fell) atomicAdd(fallbacks, fell);
}

enum class Simple { Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, MXFP4, NVFP4 };

template <Simple K> struct SimpleGeom;
template <> struct SimpleGeom<Simple::Q8_0> { static constexpr int BYTES = 34; };   // bytes per 32 elements
template <> struct SimpleGeom<Simple::Q4_0> { static constexpr int BYTES = 18; };
template <> struct SimpleGeom<Simple::Q4_1> { static constexpr int BYTES = 20; };
template <> struct SimpleGeom<Simple::Q5_0> { static constexpr int BYTES = 22; };
template <> struct SimpleGeom<Simple::Q5_1> { static constexpr int BYTES = 24; };
template <> struct SimpleGeom<Simple::MXFP4> { static constexpr int BYTES = 17; };
template <> struct SimpleGeom<Simple::NVFP4> { static constexpr int BYTES = 18; };  // half of a 64-element block
template <Simple K> constexpr int kBytesPer4Runs = 4 * SimpleGeom<K>::BYTES;

GGUF_D void st16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
GGUF_D void st32(uint8_t *p, uint32_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); p[2] = (uint8_t)(v >> 16); p[3] = (uint8_t)(v >> 24); }

// (int8_t)(float) as the x86 build of upstream does it: truncation to int32 with out-of-range
// values and NaN giving INT_MIN, then the low byte.
GGUF_D int trunc_to_i8(float v) {
    const int i = fabsf(v) < 2147483648.f ? __float2int_rz(v) : (int)0x80000000;
    return (int)(int8_t)(i & 0xFF);
}

// roundf (halves away from zero) for |v| < 2^23 without the library call
GGUF_D int round_half_away(float v) {
    const float t = truncf(v);
    const float frac = v - t;  // exact
    return (int)t + (frac >= 0.5f ? 1 : 0) - (frac <= -0.5f ? 1 : 0);
}

constexpr int kBlockThreads = 128;   // one thread per 32 elements
constexpr int kRowStride = 36;       // floats per staged 32-element run: 16-byte aligned rows, conflict-free LDS.128
constexpr float kInf = kInfinity;

// Three-input extrema (sm_100): max(|a|,|b|,|c|) returning NaN when any input is NaN, and the
// plain three-input max / min, which skip NaN inputs like upstream's `if (v > max)` loops do.
GGUF_D float amax3_nan(float a, float b, float c) {
    float d;
    asm("max.NaN.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
GGUF_D float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
GGUF_D float min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// max |x[0..N)|, NaN if any element is NaN
template <int N>
GGUF_D float amax_nan(const float *x) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < N; j += 2) m = amax3_nan(m, x[j], x[j + 1]);
    return m;
}

// floor(v) for 0 <= v < 2^23 in the low mantissa bits of the result: the sum v + 2^23 is rounded down.
GGUF_D uint32_t floor_bits(float v) { return __float_as_uint(__fadd_rd(v, 8388608.f)); }
// low bytes of a and b -> 16 bits
GGUF_D uint32_t pack2(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x0040); }

// `nhalf` 16-bit units to a shared-memory address that is 2-byte aligned when `even` is set.
template <int NHALF>
GGUF_D void emit_halves(uint8_t *out, const uint32_t (&h)[NHALF], bool even) {
    if (even) {
#pragma unroll
        for (int i = 0; i < NHALF; ++i) reinterpret_cast<uint16_t *>(out)[i] = (uint16_t)h[i];
    } else {
#pragma unroll
        for (int i = 0; i < NHALF; ++i) st16(out + 2 * i, (uint16_t)h[i]);
    }
}

// MXFP4 scale byte: (uint8_t)(floorf(log2f(amax)) - 2 + 127) as the x86 build computes it.
// `mx_steps`: per binade [2^t, 2^(t+1)), t = -149..127, the smallest float for which the host libm's
// floorf(log2f(x)) already returns t+1 (+inf bits if it never does).
GGUF_D int mxfp4_scale_byte(float amax, const float *__restrict__ mx_steps) {
    if (!(amax > 0.0f)) return 0;
    const uint32_t bits = f32_to_bits(amax);
    const int bexp = (int)(bits >> 23);  // 255 (inf) converts to 0x80000000 on x86: low byte 0
    const int t = bexp ? bexp - 127 : (31 - __clz((int)(bits & 0x7fffffu))) - 149;
    const int fl = (t >= -149 && t <= 127 && amax >= mx_steps[t + 149]) ? t + 1 : t;
    return bexp == 255 ? 0 : (fl - 2 + 127) & 0xFF;
}

// The encoders as upstream writes them, element by element from the staged run in shared memory,
// rolled loops, byte stores.  They serve every input the fast encoders decline (non-finite values,
// scales whose reciprocal overflows, sign-of-zero and first-of-equal-extrema questions).
template <Simple K>
__device__ __noinline__ void encode_exact(const float *x, uint8_t *out, const float *__restrict__ mx_steps) {
    if constexpr (K == Simple::Q8_0) {
        // upstream q8_0.cpp:16-43; MAX(a, b) = a > b ? a : b forgets the running maximum at a NaN
        float amax = 0.0f;
#pragma unroll 1
        for (int j = 0; j < 32; ++j) { const float a = fabsf(x[j]); amax = amax > a ? amax : a; }
        const float d = amax / 127.0f;
        const float id = d ? 1.0f / d : 0.0f;
        st16(out, f32_to_half_bits(d));
#pragma unroll 1
        for (int j = 0; j < 32; ++j) {
            const float v = x[j] * id;
            // (int8_t)roundf(v): out-of-range and NaN convert to INT_MIN, low byte 0
            out[2 + j] = fabsf(v) < 2147483648.f ? (uint8_t)(int8_t)round_half_away(v) : (uint8_t)0;
        }
    } else if constexpr (K == Simple::Q4_0 || K == Simple::Q5_0) {
        // upstream q4_0.cpp:16-58, q5_0.cpp:18-65
        constexpr bool FIVE = K == Simple::Q5_0;
        float amax = 0.0f, vmax = 0.0f;
#pragma unroll 1
        for (int j = 0; j < 32; ++j) {
            if (amax < fabsf(x[j])) { amax = fabsf(x[j]); vmax = x[j]; }
        }
        const float d = vmax / (FIVE ? -16.0f : -8.0f);
        const float id = d ? 1.0f / d : 0.0f;
        st16(out, f32_to_half_bits(d));
        uint32_t qh = 0;
#pragma unroll 1
        for (int j = 0; j < 16; ++j) {
            const int q0 = imin(FIVE ? 31 : 15, trunc_to_i8(x[j] * id + (FIVE ? 16.5f : 8.5f))) & 0xFF;
            const int q1 = imin(FIVE ? 31 : 15, trunc_to_i8(x[j + 16] * id + (FIVE ? 16.5f : 8.5f))) & 0xFF;
            if (FIVE) {
                out[6 + j] = (uint8_t)((q0 & 0x0F) | ((q1 & 0x0F) << 4));
                qh |= (uint32_t)((q0 & 0x10) >> 4) << j;
                qh |= (uint32_t)((q1 & 0x10) >> 4) << (j + 16);
            } else {
                out[2 + j] = (uint8_t)(q0 | (q1 << 4));
            }
        }
        if (FIVE) st32(out + 2, qh);
    } else if constexpr (K == Simple::Q4_1 || K == Simple::Q5_1) {
        // upstream q4_1.cpp:16-57, q5_1.cpp:18-68
        constexpr bool FIVE = K == Simple::Q5_1;
        float mn = FLT_MAX, mx = -FLT_MAX;
#pragma unroll 1
        for (int j = 0; j < 32; ++j) {
            if (x[j] < mn) mn = x[j];
            if (x[j] > mx) mx = x[j];
        }
        const float d = (mx - mn) / (FIVE ? 31.0f : 15.0f);
        const float id = d ? 1.0f / d : 0.0f;
        st16(out, f32_to_half_bits(d));
        st16(out + 2, f32_to_half_bits(mn));
        uint32_t qh = 0;
#pragma unroll 1
        for (int j = 0; j < 16; ++j) {
            const float t0 = (x[j] - mn) * id + 0.5f, t1 = (x[j + 16] - mn) * id + 0.5f;
            if (FIVE) {
                // (uint8_t)(float): truncation through int32, low byte
                const int q0 = (fabsf(t0) < 2147483648.f ? __float2int_rz(t0) : (int)0x80000000) & 0xFF;
                const int q1 = (fabsf(t1) < 2147483648.f ? __float2int_rz(t1) : (int)0x80000000) & 0xFF;
                out[8 + j] = (uint8_t)((q0 & 0x0F) | ((q1 & 0x0F) << 4));
                qh |= (uint32_t)((q0 & 0x10) >> 4) << j;
                qh |= (uint32_t)((q1 & 0x10) >> 4) << (j + 16);
            } else {
                const int q0 = imin(15, trunc_to_i8(t0)) & 0xFF, q1 = imin(15, trunc_to_i8(t1)) & 0xFF;
                out[4 + j] = (uint8_t)(q0 | (q1 << 4));
            }
        }
        if (FIVE) st32(out + 4, qh);
    } else if constexpr (K == Simple::MXFP4) {
        // upstream mxfp4.cpp:17-54
        float amax = 0.0f;
#pragma unroll 1
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
        const int e = mxfp4_scale_byte(amax, mx_steps);
        const float d = e8m0_half_to_f32((uint8_t)e);
        out[0] = (uint8_t)e;
#pragma unroll 1
        for (int j = 0; j < 16; ++j) out[1 + j] = (uint8_t)(best_index_fp4(x[j], d) | (best_index_fp4(x[j + 16], d) << 4));
    }
}

// One 16-element NVFP4 sub-block the way upstream writes it (nvfp4.cpp:28-54).
__device__ __noinline__ void encode_exact_nvfp4(const float *x, uint8_t *scale_byte, uint8_t *qs) {
    float amax = 0.0f;
#pragma unroll 1
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const uint8_t ue = f32_to_ue4m3(amax / 6.0f);
    const float d = ue4m3_half_to_f32(ue);
    *scale_byte = ue;
#pragma unroll 1
    for (int j = 0; j < 8; ++j) qs[j] = (uint8_t)(best_index_fp4(x[j], d) | (best_index_fp4(x[j + 8], d) << 4));
}

// 16-byte asynchronous copy global -> shared (LDGSTS), bypassing L1 and the register file.
GGUF_D void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
GGUF_D void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
GGUF_D void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// 32-element types (and NVFP4 as two 16-element sub-blocks per thread).  Persistent CTAs walk the
// tiles (128 runs of 32 floats) with a stride of the grid size.  A tile is staged in shared memory
// by coalesced 16-byte asynchronous copies, one tile ahead of the one being encoded, so the copy of
// tile i+1 is in flight while every thread encodes its own 32 elements of tile i from registers; the
// encoded tile is written out as 16-byte vectors.
template <Simple K>
__global__ void __launch_bounds__(kBlockThreads) quant32_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                               int64_t nruns, const float *__restrict__ mx_steps) {
    constexpr int BYTES = SimpleGeom<K>::BYTES;
    __shared__ __align__(16) float xbuf[2][kBlockThreads * kRowStride];
    constexpr int BYTES4 = kBytesPer4Runs<K>;
    __shared__ __align__(16) uint8_t stage[kBlockThreads / 4 * BYTES4 + 32];

    const int64_t ntiles = (nruns + kBlockThreads - 1) / kBlockThreads;
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15);  // a tile starts a multiple of 16 bytes into dst
    uint8_t *tile = stage + mis;
    const bool even = (mis & 1) == 0, word_aligned = (mis & 3) == 0;

    auto prefetch = [&](int64_t t, float *xin) {
        const int64_t r0 = t * kBlockThreads;
        const int nr = (int)(nruns - r0 < kBlockThreads ? nruns - r0 : kBlockThreads);
        const float4 *g4 = reinterpret_cast<const float4 *>(src + r0 * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = k * kBlockThreads + threadIdx.x;  // float4 index inside the tile
            if (i < nr * 8) cp_async16(xin + (i >> 3) * kRowStride + (i & 7) * 4, g4 + i);
        }
        cp_async_commit();
    };

    int64_t t = blockIdx.x;
    grid_dependents_may_launch();
    grid_dependency_wait();
    if (t < ntiles) prefetch(t, xbuf[0]);
    for (int it = 0; t < ntiles; t += gridDim.x, ++it) {
    float *xin = xbuf[it & 1];
    const int64_t tnext = t + gridDim.x;
    if (tnext < ntiles) {
        prefetch(tnext, xbuf[(it + 1) & 1]);
        cp_async_wait<1>();
    } else {
        cp_async_wait<0>();
    }
    __syncthreads();  // tile t is in xin; every thread is done with the previous tile's stage
    const int64_t r0 = t * kBlockThreads;
    const int nr = (int)(nruns - r0 < kBlockThreads ? nruns - r0 : kBlockThreads);
    uint8_t *gdst = dst + r0 / 4 * BYTES4;   // r0 is a multiple of 128
    if (threadIdx.x < nr) {
        const float *xrow = xin + threadIdx.x * kRowStride;
        float x[32];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 v = *reinterpret_cast<const float4 *>(xrow + 4 * k);
            x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
        }
        uint8_t *out = tile + threadIdx.x * BYTES;
        if constexpr (K == Simple::Q8_0) {
            const float amax = amax_nan<32>(x);
            const float d = amax / 127.0f;
            const float id = d ? 1.0f / d : 0.0f;
            if (amax < kInf && id < kInf) {
                // |x * id| <= 127.00002: roundf(v) = sign(v) * floor(|v| + 0.5); the first sum rounded down
                // has the same floor as the exact sum.
                uint32_t h[17];
                h[0] = f32_to_half_bits(d);
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float v0 = x[j] * id, v1 = x[j + 1] * id;
                    int q0 = (int)floor_bits(__fadd_rd(fabsf(v0), 0.5f)), q1 = (int)floor_bits(__fadd_rd(fabsf(v1), 0.5f));
                    if (v0 < 0.f) q0 = -q0;
                    if (v1 < 0.f) q1 = -q1;
                    h[1 + j / 2] = pack2((uint32_t)q0, (uint32_t)q1);
                }
                emit_halves(out, h, even);
            } else {
                encode_exact<K>(xrow, out, mx_steps);
            }
        } else if constexpr (K == Simple::Q4_0 || K == Simple::Q5_0) {
            constexpr bool FIVE = K == Simple::Q5_0;
            // the element of largest magnitude is the largest or the smallest element; when both have that
            // magnitude (or all are zero) upstream takes the first one, which the exact encoder finds
            float hi = -kInf, lo = kInf;
#pragma unroll
            for (int j = 0; j < 32; j += 2) { hi = max3(hi, x[j], x[j + 1]); lo = min3(lo, x[j], x[j + 1]); }
            const float vmax = hi > -lo ? hi : lo;
            const float d = vmax / (FIVE ? -16.0f : -8.0f);
            const float id = d ? 1.0f / d : 0.0f;
            if (hi != -lo && fabsf(id) < kInf) {
                // x * id + 8.5 lies in [0.49, 16.51] (NaN for a NaN element, which upstream stores as 0):
                // (int8_t) truncation = floor, MIN(15, .) = the upper clamp
                constexpr float OFF = FIVE ? 16.5f : 8.5f, TOP = FIVE ? 31.75f : 15.75f;
                constexpr int HEAD = FIVE ? 3 : 1;
                uint32_t h[HEAD + 8];
                h[0] = f32_to_half_bits(d);
                uint32_t qh = 0;
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    uint32_t b[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint32_t a0 = floor_bits(fminf(fmaxf(x[j + k] * id + OFF, 0.f), TOP));
                        const uint32_t a1 = floor_bits(fminf(fmaxf(x[j + k + 16] * id + OFF, 0.f), TOP));
                        if (FIVE) {
                            qh |= ((a0 >> 4) & 1u) << (j + k);
                            qh |= ((a1 >> 4) & 1u) << (j + k + 16);
                            b[k] = (a0 & 0xFu) + (a1 << 4);
                        } else {
                            b[k] = a0 + (a1 << 4);  // only the low byte is kept
                        }
                    }
                    h[HEAD + j / 2] = pack2(b[0], b[1]);
                }
                if (FIVE) { h[1] = qh & 0xFFFFu; h[2] = qh >> 16; }
                emit_halves(out, h, even);
            } else {
                encode_exact<K>(xrow, out, mx_steps);
            }
        } else if constexpr (K == Simple::Q4_1 || K == Simple::Q5_1) {
            constexpr bool FIVE = K == Simple::Q5_1;
            float mx = -FLT_MAX, mn = FLT_MAX;
#pragma unroll
            for (int j = 0; j < 32; j += 2) { mx = max3(mx, x[j], x[j + 1]); mn = min3(mn, x[j], x[j + 1]); }
            const float d = (mx - mn) / (FIVE ? 31.0f : 15.0f);
            const float id = d ? 1.0f / d : 0.0f;
            // a zero extremum may be +0 or -0 depending on which came first: left to the exact encoder
            if (mn != 0.f && mx != 0.f && id < kInf) {
                constexpr float TOP = FIVE ? 31.75f : 15.75f;
                constexpr int HEAD = FIVE ? 4 : 2;
                uint32_t h[HEAD + 8];
                h[0] = f32_to_half_bits(d);
                h[1] = f32_to_half_bits(mn);
                uint32_t qh = 0;
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    uint32_t b[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint32_t a0 = floor_bits(fminf(fmaxf((x[j + k] - mn) * id + 0.5f, 0.f), TOP));
                        const uint32_t a1 = floor_bits(fminf(fmaxf((x[j + k + 16] - mn) * id + 0.5f, 0.f), TOP));
                        if (FIVE) {
                            qh |= ((a0 >> 4) & 1u) << (j + k);
                            qh |= ((a1 >> 4) & 1u) << (j + k + 16);
                            b[k] = (a0 & 0xFu) + (a1 << 4);
                        } else {
                            b[k] = a0 + (a1 << 4);
                        }
                    }
                    h[HEAD + j / 2] = pack2(b[0], b[1]);
                }
                if (FIVE) { h[2] = qh & 0xFFFFu; h[3] = qh >> 16; }
                emit_halves(out, h, even);
            } else {
                encode_exact<K>(xrow, out, mx_steps);
            }
        } else if constexpr (K == Simple::MXFP4) {
            const float amax = amax_nan<32>(x);
            const int e = mxfp4_scale_byte(amax, mx_steps);
            const float d = e8m0_half_to_f32((uint8_t)e);
            if (amax < kInf && e <= 252 && fp4_thresholds_valid(amax, d)) {
                const float scale_rz = mx_scale_rz(e);
                out[0] = (uint8_t)e;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    float lo[4], hi[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { lo[i] = mx_nudge(x[4 * w + i], scale_rz); hi[i] = mx_nudge(x[4 * w + i + 16], scale_rz); }
                    st32(out + 1 + 4 * w, drop_negative_zero(cvt_e2m1x8(lo, hi)));
                }
            } else {
                encode_exact<K>(xrow, out, mx_steps);
            }
        } else {
            // NVFP4, upstream nvfp4.cpp:16-55: this thread's 32 elements are sub-blocks 2h and 2h+1 of the
            // 64-element block blk, whose 36 bytes are 4 scale bytes followed by 4 x 8 quant bytes.
            uint8_t *blk = tile + (threadIdx.x >> 1) * 36;
            const int h = threadIdx.x & 1;
#pragma unroll
            for (int sb = 0; sb < 2; ++sb) {
                const float *xs = x + 16 * sb;
                uint8_t *scale_byte = blk + 2 * h + sb, *qs = blk + 4 + 16 * h + 8 * sb;
                const float amax = amax_nan<16>(xs);
                bool done = false;
                if (amax < kInf) {
                    const uint8_t ue = f32_to_ue4m3(amax / 6.0f);
                    const float d = ue4m3_half_to_f32(ue);
                    if (fp4_thresholds_valid(amax, d)) {
                        const Fp4Bracket k = fp4_bracket(d);
                        uint32_t other[2], words[2];
#pragma unroll
                        for (int w = 0; w < 2; ++w) words[w] = fp4_word_bracketed(xs + 4 * w, xs + 4 * w + 8, k, other[w]);
                        if (other[0] | other[1]) {
#pragma unroll
                            for (int w = 0; w < 2; ++w) words[w] = fp4_settle(words[w], other[w], xrow + 16 * sb, w, d);
                        }
                        *scale_byte = ue;
                        if (word_aligned) {
                            reinterpret_cast<uint32_t *>(qs)[0] = words[0];
                            reinterpret_cast<uint32_t *>(qs)[1] = words[1];
                        } else {
                            st32(qs, words[0]);
                            st32(qs + 4, words[1]);
                        }
                        done = true;
                    }
                }
                if (!done) encode_exact_nvfp4(xrow + 16 * sb, scale_byte, qs);
            }
        }
    }
    __syncthreads();
    flush_tile(tile, gdst, nr * BYTES4 / 4, threadIdx.x, kBlockThreads);
    }
}

// lroundf(x * id) + 1.  With a finite id the product lies in [-1, 1] (or is NaN, which upstream's
// conversion turns into digit 1) and rounding half away from zero is two comparisons.  When the
// scale is so small that 1 / d overflows (or d is NaN) every product is an infinity or NaN, which
// x86's conversion turns into the integer indefinite value 0x8000...0: digit 1 after the increment.
GGUF_D uint32_t trit(float x, float id) {
    const float v = x * id;
    return 1u + (v >= 0.5f ? 1u : 0u) - (v <= -0.5f ? 1u : 0u);
}
// five base-3 digits (most significant first) -> TQ1_0's byte: ceil(q * 256 / 243)
GGUF_D uint32_t tq1_byte(uint32_t q) { return (q * 256u + 242u) / 243u; }

constexpr int kTernThreads = 128;               // eight lanes per block
constexpr int kTernBlocks = kTernThreads / 8;   // blocks per tile

// Copies that did not land within the wait limit, all launches of this process on the device.
__device__ unsigned long long g_staging_timeouts;
// try_wait rounds a consumer spends on a staged tile before it gives up.  The host can lower it (down to 0: give up
// at once) so that the give-up path can be exercised without a copy that is really lost; the drain waits keep the
// full limit.
__device__ int g_staging_wait_limit = kBulkWaitLimit;

// TQ1_0 / TQ2_0: 256-element blocks, d = max |x| (upstream tq1_0.cpp:16-98, tq2_0.cpp:16-53).
// Persistent CTAs walk tiles of sixteen blocks (16 KB, contiguous) with a stride of the grid size; one thread
// stages tile i+1 with a single bulk asynchronous copy while tile i is encoded.  Eight lanes share a block: every
// output byte mixes elements 32 (or 16, or 4) apart, and lane L takes the elements of bytes 4L..4L+3 of each
// 32-byte group (TQ1_0: also bytes 32+2L, 33+2L and, for L < 4, byte 48+L) straight from the staged block, 30 to 34
// elements in registers.  The encoded tile leaves as 16-byte vectors.
template <bool TQ1>
__global__ void __launch_bounds__(kTernThreads) quant_ternary_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                                    int64_t nblocks) {
    constexpr int BYTES = TQ1 ? 54 : 66;
    __shared__ __align__(128) float xs[2][kTernBlocks * 256];
    __shared__ __align__(16) uint8_t stage[kTernBlocks * BYTES + 16];
    __shared__ __align__(8) uint64_t landed[2];
    const int group = threadIdx.x >> 3, L = threadIdx.x & 7;
    const int64_t ntiles = (nblocks + kTernBlocks - 1) / kTernBlocks;
    uint8_t *tile = stage + (reinterpret_cast<uintptr_t>(dst) & 15);  // a tile starts a multiple of 16 bytes into dst

    if (threadIdx.x == 0) {
        mbarrier_init(&landed[0], 1);
        mbarrier_init(&landed[1], 1);
        fence_async_shared();
    }
    __syncthreads();
    // thread 0 only; every thread has passed a barrier since it last read the slot
    auto prefetch = [&](int64_t t, int slot) {
        const int64_t left = nblocks - t * kTernBlocks;
        const uint32_t bytes = (uint32_t)(left < kTernBlocks ? left : kTernBlocks) * 1024u;
        fence_async_shared();
        bulk_load(xs[slot], src + t * kTernBlocks * 256, bytes, &landed[slot]);
    };

    int64_t t = blockIdx.x;
    grid_dependents_may_launch();
    grid_dependency_wait();
    const int wait_limit = g_staging_wait_limit;
    if (t < ntiles && threadIdx.x == 0) prefetch(t, 0);
    for (int it = 0; t < ntiles; t += gridDim.x, ++it) {
        const int64_t tnext = t + gridDim.x;
        if (tnext < ntiles && threadIdx.x == 0) prefetch(tnext, (it + 1) & 1);
        // slot it & 1 is on its (it / 2)-th use: wait for that phase
        const bool arrived = mbarrier_wait(&landed[it & 1], (uint32_t)(it >> 1) & 1u, wait_limit);
        // also orders the previous tile's flush before this tile's writes to the stage
        if (!__syncthreads_and(arrived)) {
            // Gave up: no further copies are issued.  Two may still be in flight, this tile's and the next one's;
            // each gets one more bounded wait before the CTA leaves its shared memory behind.
            mbarrier_wait(&landed[it & 1], (uint32_t)(it >> 1) & 1u);
            if (tnext < ntiles) mbarrier_wait(&landed[(it + 1) & 1], (uint32_t)((it + 1) >> 1) & 1u);
            if (threadIdx.x == 0) atomicAdd(&g_staging_timeouts, 1ull);
            return;
        }
        const int64_t first = t * kTernBlocks;
        const float *xb = xs[it & 1] + group * 256;
        // Groups past the end of a short last tile run on stale data (all lanes take part in the shuffles) and store nothing.
        const bool live = first + group < nblocks;
        constexpr int N = TQ1 ? 36 : 32;
        float x[N];
        if constexpr (TQ1) {
#pragma unroll
            for (int n = 0; n < 5; ++n) {
                const float4 v = *reinterpret_cast<const float4 *>(xb + n * 32 + 4 * L);
                x[4 * n] = v.x; x[4 * n + 1] = v.y; x[4 * n + 2] = v.z; x[4 * n + 3] = v.w;
                const float2 w = *reinterpret_cast<const float2 *>(xb + 160 + n * 16 + 2 * L);
                x[20 + 2 * n] = w.x; x[21 + 2 * n] = w.y;
            }
#pragma unroll
            for (int n = 0; n < 4; ++n) x[30 + n] = L < 4 ? xb[240 + n * 4 + L] : 0.f;
            x[34] = x[35] = 0.f;
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {  // k = 4 * group-of-128 + n
                const float4 v = *reinterpret_cast<const float4 *>(xb + k * 32 + 4 * L);
                x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
            }
        }
        float amax = amax_nan<N>(x);
#pragma unroll
        for (int m = 4; m > 0; m >>= 1) {
            const float other = __shfl_xor_sync(kFull, amax, m);
            amax = amax3_nan(amax, other, other);
        }
        if (amax != amax) {
            // upstream's MAX(a, b) = a > b ? a : b forgets the running maximum at a NaN: redo its loop in element order
            float a = 0.f;
            for (int i = 0; i < 256; ++i) {
                const float m = fabsf(xb[i]);
                a = a > m ? a : m;
            }
            amax = a;
        }
        const float d = amax;
        const float id = d ? 1.0f / d : 0.0f;
        const bool finite = id < kInfinity;   // otherwise every digit is 1
        uint8_t *out = tile + group * BYTES;
        if (live) {
            if constexpr (TQ1) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t q = 0;
#pragma unroll
                    for (int n = 0; n < 5; ++n) q = q * 3u + trit(x[4 * n + c], id);
                    out[4 * L + c] = (uint8_t)tq1_byte(finite ? q : 121u);
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t q = 0;
#pragma unroll
                    for (int n = 0; n < 5; ++n) q = q * 3u + trit(x[20 + 2 * n + c], id);
                    out[32 + 2 * L + c] = (uint8_t)tq1_byte(finite ? q : 121u);
                }
                if (L < 4) {
                    uint32_t q = 0;
#pragma unroll
                    for (int n = 0; n < 4; ++n) q = q * 3u + trit(x[30 + n], id);
                    out[48 + L] = (uint8_t)tq1_byte(finite ? q * 3u : 120u);
                }
                if (L == 0) st16(out + 52, f32_to_half_bits(d));
            } else {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t q = 0;
#pragma unroll
                        for (int n = 0; n < 4; ++n) q |= trit(x[4 * (4 * j + n) + c], id) << (2 * n);
                        out[32 * j + 4 * L + c] = (uint8_t)(finite ? q : 0x55u);
                    }
                }
                if (L == 0) st16(out + 64, f32_to_half_bits(d));
            }
        }
        __syncthreads();
        const int64_t left = nblocks - first;
        flush_tile(tile, dst + first * BYTES, (int)(left < kTernBlocks ? left : kTernBlocks) * BYTES, threadIdx.x, kTernThreads);
    }
}

template <bool TQ1>
cudaError_t launch_ternary(const float *src, uint8_t *dst, int64_t nblocks, cudaStream_t stream) {
    const int64_t ntiles = (nblocks + kTernBlocks - 1) / kTernBlocks;
    if (ntiles <= 0) return cudaSuccess;
    static const int resident = [] {
        int dev = 0, sms = 148, per_sm = 6;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_ternary_kernel<TQ1>, kTernThreads, 0);
        return sms * (per_sm > 0 ? per_sm : 1);
    }();
    const int64_t grid = ntiles < resident ? ntiles : resident;
    const cudaError_t launched = launch_overlapped(quant_ternary_kernel<TQ1>, (unsigned)grid, kTernThreads, stream, src, dst, nblocks);
    count_launch();
    return launched != cudaSuccess ? launched : cudaGetLastError();
}

// Q1_0, upstream q1_0.cpp:16-55: d = (sum of |x| over the block's 128 elements, added in element order) / 128, one
// bit per element (x >= 0).  The sum is a chain of 128 dependent additions, so a lane owns a whole block: one-warp
// CTAs walk tiles of 32 blocks; every lane stages its own block (512 bytes) with one bulk asynchronous copy into a
// row padded to 132 floats (16-byte aligned, conflict-free 16-byte reads), one tile ahead of the one being encoded.
// Four lanes per block, the sum handed from lane to lane, executed the chain four times over and ran at 81 %.
constexpr int kQ1Stride = 132;
__global__ void __launch_bounds__(32) quant_q1_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst, int64_t nblocks) {
    constexpr int BYTES = 18;
    __shared__ __align__(128) float xs[2][32 * kQ1Stride];
    __shared__ __align__(16) uint8_t stage[32 * BYTES + 16];
    __shared__ __align__(8) uint64_t landed[2];
    const int lane = threadIdx.x;
    const int64_t ntiles = (nblocks + 31) / 32;
    uint8_t *tile = stage + (reinterpret_cast<uintptr_t>(dst) & 15);  // a tile starts a multiple of 16 bytes into dst
    if (lane == 0) {
        mbarrier_init(&landed[0], 32);
        mbarrier_init(&landed[1], 32);
        fence_async_shared();
    }
    __syncwarp();
    // A lane overwrites the row it read itself during the slot's previous use, hence only the proxy fence.
    auto prefetch = [&](int64_t t, int slot) {
        const int64_t b = t * 32 + lane;
        if (b < nblocks) {
            fence_async_shared();
            bulk_load(xs[slot] + lane * kQ1Stride, src + b * 128, 512u, &landed[slot]);
        } else {
            mbarrier_arrive(&landed[slot]);
        }
    };

    int64_t t = blockIdx.x;
    grid_dependents_may_launch();
    grid_dependency_wait();
    const int wait_limit = g_staging_wait_limit;
    if (t < ntiles) prefetch(t, 0);
    for (int it = 0; t < ntiles; t += gridDim.x, ++it) {
        const int64_t tnext = t + gridDim.x;
        if (tnext < ntiles) prefetch(tnext, (it + 1) & 1);
        const bool arrived = mbarrier_wait(&landed[it & 1], (uint32_t)(it >> 1) & 1u, wait_limit);
        if (!__all_sync(kFull, arrived)) {
            // as in the ternary kernel: stop, wait once more (bounded) for the copies of both slots, then leave
            mbarrier_wait(&landed[it & 1], (uint32_t)(it >> 1) & 1u);
            if (tnext < ntiles) mbarrier_wait(&landed[(it + 1) & 1], (uint32_t)((it + 1) >> 1) & 1u);
            if (lane == 0) atomicAdd(&g_staging_timeouts, 1ull);
            return;
        }
        const float *row = xs[it & 1] + lane * kQ1Stride;
        float total = 0.f;
        uint32_t bits[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float4 v = *reinterpret_cast<const float4 *>(row + 32 * w + 4 * k);
                total += fabsf(v.x); total += fabsf(v.y); total += fabsf(v.z); total += fabsf(v.w);
                word |= (v.x >= 0.0f ? 1u : 0u) << (4 * k) | (v.y >= 0.0f ? 1u : 0u) << (4 * k + 1) |
                        (v.z >= 0.0f ? 1u : 0u) << (4 * k + 2) | (v.w >= 0.0f ? 1u : 0u) << (4 * k + 3);
            }
            bits[w] = word;
        }
        const int64_t first = t * 32;
        if (first + lane < nblocks) {  // lanes past the end of a short last tile worked on stale rows
            uint8_t *out = tile + lane * BYTES;
            st16(out, f32_to_half_bits(total / 128.0f));
#pragma unroll
            for (int w = 0; w < 4; ++w) st32(out + 2 + 4 * w, bits[w]);
        }
        __syncwarp();
        const int64_t left = nblocks - first;
        flush_tile(tile, dst + first * BYTES, (int)(left < 32 ? left : 32) * BYTES, lane, 32);
        __syncwarp();  // the flush has read the stage before the next tile's blocks are written to it
    }
}

cudaError_t launch_q1(const float *src, uint8_t *dst, int64_t nblocks, cudaStream_t stream) {
    const int64_t ntiles = (nblocks + 31) / 32;
    if (ntiles <= 0) return cudaSuccess;
    static const int resident = [] {
        int dev = 0, sms = 148, per_sm = 6;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_q1_kernel, 32, 0);
        return sms * (per_sm > 0 ? per_sm : 1);
    }();
    const int64_t grid = ntiles < resident ? ntiles : resident;
    const cudaError_t launched = launch_overlapped(quant_q1_kernel, (unsigned)grid, 32, stream, src, dst, nblocks);
    count_launch();
    return launched != cudaSuccess ? launched : cudaGetLastError();
}

// Plain storage types: fp32 copy, fp16 and bf16 conversion with upstream's rounding and NaN
// handling (upstream libgguf_storage.cpp:105-125).  kind: 0 copy, 1 fp16, 2 bf16.
template <int KIND>
__global__ void __launch_bounds__(kThreads) store_kernel(const float *__restrict__ src, void *__restrict__ dst, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float v = src[i];
        if (KIND == 0) static_cast<float *>(dst)[i] = v;
        else if (KIND == 1) static_cast<uint16_t *>(dst)[i] = f32_to_half_bits(v);
        else static_cast<uint16_t *>(dst)[i] = f32_to_bf16_bits(v);
    }
}

template <Simple K>
cudaError_t launch32(const float *src, void *dst, int64_t nelems, const float *mx_steps, cudaStream_t stream) {
    const int64_t nruns = nelems / 32;
    const int64_t ntiles = (nruns + kBlockThreads - 1) / kBlockThreads;
    if (ntiles <= 0) return cudaSuccess;
    // persistent CTAs: as many as can be resident (5 per SM by shared memory), fewer for small inputs
    static const int resident = [] {
        int dev = 0, sms = 148, per_sm = 5;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant32_kernel<K>, kBlockThreads, 0);
        return sms * (per_sm > 0 ? per_sm : 1);
    }();
    const int64_t grid = ntiles < resident ? ntiles : resident;
    const cudaError_t launched = launch_overlapped(quant32_kernel<K>, (unsigned)grid, kBlockThreads, stream, src,
                                                   static_cast<uint8_t *>(dst), nruns, mx_steps);
    count_launch();
    return launched != cudaSuccess ? launched : cudaGetLastError();
}

}  // namespace

cudaError_t read_staging_timeouts(unsigned long long *count) {
    return cudaMemcpyFromSymbol(count, g_staging_timeouts, sizeof(*count));
}

cudaError_t set_staging_wait_limit(int limit) {
    const int value = limit < 0 ? kBulkWaitLimit : limit;
    return cudaMemcpyToSymbol(g_staging_wait_limit, &value, sizeof(value));
}

bool uses_bulk_staging(int type) { return type == GGML_TYPE_TQ1_0 || type == GGML_TYPE_TQ2_0 || type == GGML_TYPE_Q1_0; }

cudaError_t launch_store(int type, const float *src, void *dst, int64_t nelems, cudaStream_t stream) {
    if (nelems <= 0) return cudaSuccess;
    int64_t grid = (nelems + kThreads - 1) / kThreads;
    if (grid > 148 * 32) grid = 148 * 32;
    switch (type) {
        case GGML_TYPE_F32: store_kernel<0><<<(unsigned)grid, kThreads, 0, stream>>>(src, dst, nelems); break;
        case GGML_TYPE_F16: store_kernel<1><<<(unsigned)grid, kThreads, 0, stream>>>(src, dst, nelems); break;
        case GGML_TYPE_BF16: store_kernel<2><<<(unsigned)grid, kThreads, 0, stream>>>(src, dst, nelems); break;
        default: return cudaErrorInvalidValue;
    }
    count_launch();
    return cudaGetLastError();
}

// Counts the inputs (all 2^32 float bit patterns) for which a fast form of the FP4 level search
// differs from the 16-way scan at scale e; counters[0] = mismatches, counters[1] = fallbacks.
cudaError_t selftest_fp4(float e, int mode, int ebyte, unsigned long long *device_counters, cudaStream_t stream) {
    selftest_fp4_kernel<<<148 * 8, 256, 0, stream>>>(e, mode, ebyte, device_counters, device_counters + 1);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_quantize_simple(int type, const float *src, void *dst, int64_t nelems, const float *mx_steps,
                                   cudaStream_t stream) {
    uint8_t *out = static_cast<uint8_t *>(dst);
    switch (type) {
        case GGML_TYPE_Q8_0: return launch32<Simple::Q8_0>(src, dst, nelems, nullptr, stream);
        case GGML_TYPE_Q4_0: return launch32<Simple::Q4_0>(src, dst, nelems, nullptr, stream);
        case GGML_TYPE_Q4_1: return launch32<Simple::Q4_1>(src, dst, nelems, nullptr, stream);
        case GGML_TYPE_Q5_0: return launch32<Simple::Q5_0>(src, dst, nelems, nullptr, stream);
        case GGML_TYPE_Q5_1: return launch32<Simple::Q5_1>(src, dst, nelems, nullptr, stream);
        case GGML_TYPE_MXFP4: return launch32<Simple::MXFP4>(src, dst, nelems, mx_steps, stream);
        case GGML_TYPE_NVFP4: return launch32<Simple::NVFP4>(src, dst, nelems, nullptr, stream);
        case GGML_TYPE_Q1_0: return launch_q1(src, out, nelems / 128, stream);
        case GGML_TYPE_TQ1_0: return launch_ternary<true>(src, out, nelems / 256, stream);
        case GGML_TYPE_TQ2_0: return launch_ternary<false>(src, out, nelems / 256, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gguf
