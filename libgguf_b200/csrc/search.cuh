// Scale searches shared by the K-quant, legacy-weighted and IQ4 quantizers.
//
// Every search here is inherently sequential in the upstream code: later candidates depend on
// state that an accepted candidate changed (the running minimum in the affine search, the
// running best score everywhere else), and all sums are plain left-to-right fp32 accumulations.
// So one thread owns one group of N elements, keeps the group in registers and runs the search
// exactly in upstream order; parallelism comes from the number of groups, never from splitting a
// sum.  Loops over the N elements are fully unrolled (register arrays), loops over candidates
// are not.
#pragma once

#include <float.h>

#include "gguf_common.cuh"

namespace gguf {

// Values are kept 8 bits each, four per word: element i lives in word i/4, byte i%4.
template <int N>
GGUF_D void pack_levels(const float (&lf)[N], uint32_t (&L)[N / 4]) {
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
        L[k] = (uint32_t)(int)lf[4 * k] | ((uint32_t)(int)lf[4 * k + 1] << 8) | ((uint32_t)(int)lf[4 * k + 2] << 16) |
               ((uint32_t)(int)lf[4 * k + 3] << 24);
    }
}
template <int N>
GGUF_D int level_at(const uint32_t (&L)[N / 4], int i) { return (L[i >> 2] >> (8 * (i & 3))) & 0xFF; }

constexpr float kRoundMagic = 12582912.f;  // 1.5 * 2^23
constexpr float kRoundSafe = 4000000.f;    // below 2^22 the float form of nearest_int is exact

// clamp(nearest_int(v), lo, hi) as a float.  FAST uses (v + magic) - magic, which equals
// nearest_int(v) whenever |v| < 2^22; the caller proves the bound per candidate and otherwise
// asks for the integer form, which reproduces upstream's mantissa masking for any input.
template <bool FAST>
GGUF_D float round_clamp(float v, float lo, float hi) {
    if (FAST) {
        const float r = (v + kRoundMagic) - kRoundMagic;
        return fminf(fmaxf(r, lo), hi);
    } else {
        const int l = nearest_int(v);
        return (float)imax((int)lo, imin((int)hi, l));
    }
}

// Two-wide helpers for evaluating two candidates at once.  Only additions are issued as packed instructions: the
// assembler contracts a packed multiply that feeds a packed add into one fused multiply-add even when both carry an
// explicit rounding mode (unlike the scalar instructions), which would change the rounding of every product-sum here.
// Products are therefore scalar multiplies, whose results the packed adds consume unfused.
GGUF_D float2 mul2_unfused(float2 a, float2 b) { return make_float2(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y)); }
GGUF_D float2 mul2_unfused(float a, float2 b) { return make_float2(__fmul_rn(a, b.x), __fmul_rn(a, b.y)); }
GGUF_D float2 splat2(float a) { return make_float2(a, a); }
// nearest integer of both lanes for |v| < 2^22, clamped to [lo, hi]
GGUF_D float2 round_clamp2(float2 v, float lo, float hi) {
    float2 r = __fadd2_rn(__fadd2_rn(v, splat2(kRoundMagic)), splat2(-kRoundMagic));
    r.x = fminf(fmaxf(r.x, lo), hi);
    r.y = fminf(fmaxf(r.y, lo), hi);
    return r;
}

// ---------------------------------------------------------------------------------------------
// Affine search: levels 0..nmax, value = scale*level - the_min.
// upstream libgguf_common.h:574-670 (make_qkx2_quants) and :688-785 (make_qkx3_quants); with
// explicit weights the two are the same arithmetic and differ only in the parameters passed.
template <int N, bool MAD>
GGUF_D float search_scale_min(const float (&x)[N], const float (&w)[N], int nmax, float rmin, float rdelta, int nstep,
                              float &the_min, uint32_t (&L)[N / 4]) {
    float mn = x[0], mx = x[0];
    float sum_w = w[0];
    float sum_x = sum_w * x[0];
#pragma unroll
    for (int i = 1; i < N; ++i) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
        sum_w += w[i];
        sum_x += w[i] * x[i];
    }
    const float xmin = mn;  // true minimum, for the rounding bound below
    if (mn > 0) mn = 0;
    if (mx == mn) {
#pragma unroll
        for (int k = 0; k < N / 4; ++k) L[k] = 0;
        the_min = -mn;
        return 0.f;
    }
    const float fnmax = (float)nmax;
    float lf[N];
    float iscale = fnmax / (mx - mn);
    float scale = 1 / iscale;
    float best_error = 0;
    {
        // An infinite iscale makes every upstream level 0 (inf and inf*0 both fall to the lower clamp).
        const float isr = iscale > FLT_MAX ? 0.f : iscale;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            lf[i] = round_clamp<true>(isr * (x[i] - mn), 0.f, fnmax);
            float diff = scale * lf[i] + mn - x[i];
            diff = MAD ? fabsf(diff) : diff * diff;
            best_error += w[i] * diff;
        }
        pack_levels<N>(lf, L);
    }
    if (nstep < 1) {
        the_min = -mn;
        return scale;
    }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + fnmax) / (mx - mn);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        const float isr = fabsf(iscale) > FLT_MAX ? 0.f : iscale;
        const float bound = fabsf(isr) * fmaxf(fabsf(mx - mn), fabsf(xmin - mn));
        if (bound < kRoundSafe) {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                lf[i] = round_clamp<true>(isr * (x[i] - mn), 0.f, fnmax);
                const float wl = w[i] * lf[i];
                sum_l += wl;
                sum_l2 += wl * lf[i];
                sum_xl += wl * x[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                lf[i] = round_clamp<false>(iscale * (x[i] - mn), 0.f, fnmax);
                const float wl = w[i] * lf[i];
                sum_l += wl;
                sum_l2 += wl * lf[i];
                sum_xl += wl * x[i];
            }
        }
        const float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0) {
                this_min = 0;
                this_scale = sum_xl / sum_l2;
            }
            float cur_error = 0;
#pragma unroll
            for (int i = 0; i < N; ++i) {
                float diff = this_scale * lf[i] + this_min - x[i];
                diff = MAD ? fabsf(diff) : diff * diff;
                cur_error += w[i] * diff;
            }
            if (cur_error < best_error) {
                pack_levels<N>(lf, L);
                best_error = cur_error;
                scale = this_scale;
                mn = this_min;
            }
        }
    }
    the_min = -mn;
    return scale;
}

// ---------------------------------------------------------------------------------------------
// Symmetric search: levels -nmax..nmax-1 stored as level+nmax, value = scale*level.
// upstream libgguf_common.h:398-491 (make_qx_quants) with rmse_type 1.  HAS_W: explicit weights,
// otherwise w = x*x.
template <int N, bool HAS_W>
GGUF_D float search_scale_sym(const float (&x)[N], const float (&qw)[N], int nmax, uint32_t (&L)[N / 4]) {
    float max = 0, amax = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < 1e-15f) {
#pragma unroll
        for (int k = 0; k < N / 4; ++k) L[k] = 0;
        return 0.f;
    }
    const float fnmax = (float)nmax;
    const float lo = -fnmax, hi = fnmax - 1.f;
    float iscale = (float)(-nmax) / max;
    float lf[N];
    float sumlx = 0, suml2 = 0;
    // |iscale * x[i]| <= nmax + 1 here because |x[i]| <= |max|, so the float rounding form is exact.
#pragma unroll
    for (int i = 0; i < N; ++i) {
        lf[i] = round_clamp<true>(iscale * x[i], lo, hi);
        const float w = HAS_W ? qw[i] : x[i] * x[i];
        sumlx += w * x[i] * lf[i];
        suml2 += w * lf[i] * lf[i];
    }
    float best_iscale = iscale;
    float scale = suml2 ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    // The 18 candidates is = -9..-1, 1..9 do not depend on one another (only the acceptance test looks at the
    // running best), so two are evaluated at a time, their sums in the two lanes of packed adds (every lane
    // rounded like the scalar instruction), and then offered in upstream's order.
#pragma unroll 1
    for (int pair = 0; pair < 9; ++pair) {
        const int is_a = pair < 4 ? 2 * pair - 9 : (pair == 4 ? -1 : 2 * pair - 8);
        const int is_b = pair < 4 ? is_a + 1 : (pair == 4 ? 1 : is_a + 1);
        const float2 isc = make_float2(-(fnmax + 0.1f * (float)is_a) / max, -(fnmax + 0.1f * (float)is_b) / max);
        float2 slx = make_float2(0.f, 0.f), sl2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float2 l = round_clamp2(mul2_unfused(x[i], isc), lo, hi);
            const float w = HAS_W ? qw[i] : x[i] * x[i];
            slx = __fadd2_rn(slx, mul2_unfused(w * x[i], l));
            sl2 = __fadd2_rn(sl2, mul2_unfused(mul2_unfused(w, l), l));
        }
        if (sl2.x > 0 && slx.x * slx.x > best * sl2.x) {
            best_iscale = isc.x;
            scale = slx.x / sl2.x;
            best = scale * slx.x;
        }
        if (sl2.y > 0 && slx.y * slx.y > best * sl2.y) {
            best_iscale = isc.y;
            scale = slx.y / sl2.y;
            best = scale * slx.y;
        }
    }
    // Levels of the accepted candidate, recomputed once instead of stored on every acceptance.
#pragma unroll
    for (int i = 0; i < N; ++i) lf[i] = round_clamp<true>(best_iscale * x[i], lo, hi) + fnmax;
    pack_levels<N>(lf, L);
    return scale;
}

// ---------------------------------------------------------------------------------------------
// Q3_K's coordinate-descent search with w = x*x: levels -nmax..nmax-1 stored as level+nmax.
// upstream libgguf_common.h:493-572 (make_q3_quants, do_rmse = true).
template <int N>
GGUF_D float search_scale_descent(const float (&x)[N], int nmax, uint32_t (&L)[N / 4]) {
    float max = 0, amax = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < 1e-15f) {
#pragma unroll
        for (int k = 0; k < N / 4; ++k) L[k] = 0;
        return 0.f;
    }
    const float iscale = (float)(-nmax) / max;
    float lf[N];
    float sumlx = 0, suml2 = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        lf[i] = round_clamp<true>(iscale * x[i], (float)-nmax, (float)(nmax - 1));
        const float w = x[i] * x[i];
        sumlx += w * x[i] * lf[i];
        suml2 += w * lf[i] * lf[i];
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float w = x[i] * x[i];
            float slx = sumlx - w * x[i] * lf[i];
            if (slx > 0) {
                float sl2 = suml2 - w * lf[i] * lf[i];
                int new_l = nearest_int(x[i] * sl2 / slx);
                new_l = imax(-nmax, imin(nmax - 1, new_l));
                const float nl = (float)new_l;
                if (nl != lf[i]) {
                    slx += w * x[i] * nl;
                    sl2 += w * nl * nl;
                    if (sl2 > 0 && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        lf[i] = nl;
                        sumlx = slx;
                        suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (!n_changed) break;
    }
#pragma unroll
    for (int i = 0; i < N; ++i) lf[i] += (float)nmax;
    pack_levels<N>(lf, L);
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

// ---------------------------------------------------------------------------------------------
// Non-negative scale quantizer used for the per-sub-block scales and mins of the weighted
// K-quants: levels 0..nmax, value = scale*level.  upstream libgguf_common.h:787-880
// (make_qp_quants).  x, L and w live in shared memory (n = 8 or 16, one thread per call).
GGUF_D float search_scale_positive(int n, int nmax, const float *x, uint8_t *L, const float *w) {
    float max = 0;
    for (int i = 0; i < n; ++i) max = fmaxf(max, x[i]);
    if (max < 1e-15f) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.f;
    }
    float iscale = (float)nmax / max;
    for (int i = 0; i < n; ++i) L[i] = (uint8_t)nearest_int(iscale * x[i]);
    const float scale = 1 / iscale;
    float best_mse = 0;
    for (int i = 0; i < n; ++i) {
        const float diff = x[i] - scale * (float)L[i];
        best_mse += w[i] * diff * diff;
    }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        const float iscale_is = (0.1f * (float)is + (float)nmax) / max;
        const float scale_is = 1 / iscale_is;
        float mse = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale_is * x[i]);
            l = imin(nmax, l);
            const float diff = x[i] - scale_is * (float)l;
            mse += w[i] * diff * diff;
        }
        if (mse < best_mse) {
            best_mse = mse;
            iscale = iscale_is;
        }
    }
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        l = imin(nmax, l);
        L[i] = (uint8_t)l;
        sumlx += w[i] * x[i] * (float)l;
        suml2 += w[i] * (float)l * (float)l;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float wi = w[i];
            const float li = (float)L[i];
            float slx = sumlx - wi * x[i] * li;
            float sl2 = suml2 - wi * li * li;
            if (slx > 0 && sl2 > 0) {
                int new_l = nearest_int(x[i] * sl2 / slx);
                new_l = imin(nmax, new_l);
                if (new_l != (int)L[i]) {
                    slx += wi * x[i] * (float)new_l;
                    sl2 += wi * (float)new_l * (float)new_l;
                    if (slx * slx * suml2 > sumlx * sumlx * sl2) {
                        L[i] = (uint8_t)new_l;
                        sumlx = slx;
                        suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (!n_changed) break;
    }
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

}  // namespace gguf
