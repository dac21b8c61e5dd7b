// Lattice quantizers IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S.
//
// One thread owns one block of 32 (16 for IQ2_XS / IQ2_S) elements and keeps the magnitudes, the
// importance weights and their square roots in registers; the 8 or 16 threads of a super-block
// sit next to each other in a warp.  Per block the upstream algorithm is run literally: sign
// extraction (with the even-parity fix where the format stores 7 sign bits), a loop over
// candidate scales in which every group of 8 (or 4) magnitudes is rounded to the lattice and,
// when the rounded point is not a codebook entry, replaced by the best of its precomputed
// neighbours, the accept/reject chain on (sumqx, sumq2), the final re-projection, and the 4-bit
// block scale against the super-block maximum.  The codebook is staged in shared
// memory as floats (<= 32 KB) once per CTA; the lattice map and neighbour lists stay in global memory (L2 resident).
// upstream: csrc/quant/iq2_xxs.cpp:4-224, iq2_xs.cpp:4-230, iq2_s.cpp:4-218, iq3_xxs.cpp:4-273,
// iq3_s.cpp:5-233, csrc/common/libgguf_iq_tables.cpp:434-462 and :683-711.
#include <float.h>
#include <math.h>

#include "device_state.h"
#include "gguf_common.cuh"
#include "kernels.h"

namespace gguf {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kThreads = 64;

template <int TYPE> struct Traits;
template <> struct Traits<GGML_TYPE_IQ2_XXS> {
    static constexpr int BS = 32, GD = 8, BITS = 2, KMAXQ = 3, IS_MAX = 6, BYTES = 66, TABLE = IQT_2XXS;
    static constexpr bool PARITY = true, SIGMA_X2 = false, QP_INIT = true;
    static constexpr float STEP = 0.1f, EPS = 1e-15f;
};
template <> struct Traits<GGML_TYPE_IQ2_XS> {
    static constexpr int BS = 16, GD = 8, BITS = 2, KMAXQ = 3, IS_MAX = 9, BYTES = 74, TABLE = IQT_2XS;
    static constexpr bool PARITY = true, SIGMA_X2 = false, QP_INIT = false;
    static constexpr float STEP = 0.1f, EPS = 1e-15f;
};
template <> struct Traits<GGML_TYPE_IQ2_S> {
    static constexpr int BS = 16, GD = 8, BITS = 2, KMAXQ = 3, IS_MAX = 9, BYTES = 82, TABLE = IQT_2S;
    static constexpr bool PARITY = false, SIGMA_X2 = true, QP_INIT = false;
    static constexpr float STEP = 0.1f, EPS = 1e-8f;
};
template <> struct Traits<GGML_TYPE_IQ3_XXS> {
    static constexpr int BS = 32, GD = 4, BITS = 3, KMAXQ = 8, IS_MAX = 15, BYTES = 98, TABLE = IQT_3XXS;
    static constexpr bool PARITY = true, SIGMA_X2 = true, QP_INIT = false;
    static constexpr float STEP = 0.2f, EPS = 1e-8f;
};
template <> struct Traits<GGML_TYPE_IQ3_S> {
    static constexpr int BS = 32, GD = 4, BITS = 3, KMAXQ = 8, IS_MAX = 9, BYTES = 110, TABLE = IQT_3S;
    static constexpr bool PARITY = false, SIGMA_X2 = true, QP_INIT = false;
    static constexpr float STEP = 0.2f, EPS = 0.f;  // upstream tests `!max`
};

GGUF_D void st16(uint8_t *p, uint32_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
GGUF_D void st32(uint8_t *p, uint32_t v) { st16(p, v); st16(p + 2, v >> 16); }

// Levels are kept one byte each, four per register.
template <int NW>
GGUF_D int lget(const uint32_t (&L)[NW], int i) { return (int)((L[i >> 2] >> (8 * (i & 3))) & 0xFFu); }
template <int NW>
GGUF_D void lset(uint32_t (&L)[NW], int i, int v) {
    const int sh = 8 * (i & 3);
    L[i >> 2] = (L[i >> 2] & ~(0xFFu << sh)) | ((uint32_t)v << sh);
}

template <int N>
GGUF_D void load_group(const float *p, float (&x)[N]) {
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p) + k);
        x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
    }
}

// upstream libgguf_common.h:787-880 (make_qp_quants) for a group held in registers; levels
// returned one per array slot.  Only IQ2_XXS uses it (n = 32, nmax = 4).
template <int N>
GGUF_D float qp_quants_reg(int nmax, const float (&x)[N], int (&L)[N], const float (&qw)[N]) {
    float max = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) max = max > x[i] ? max : x[i];
    if (max < 1e-15f) {
#pragma unroll
        for (int i = 0; i < N; ++i) L[i] = 0;
        return 0.f;
    }
    float iscale = (float)nmax / max;
#pragma unroll
    for (int i = 0; i < N; ++i) L[i] = nearest_int(iscale * x[i]) & 0xFF;
    const float scale = 1 / iscale;
    float best_mse = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float diff = x[i] - scale * (float)L[i];
        best_mse += qw[i] * diff * diff;
    }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        const float iscale_is = (0.1f * (float)is + (float)nmax) / max;
        const float scale_is = 1 / iscale_is;
        float mse = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const int l = imin(nmax, nearest_int(iscale_is * x[i]));
            const float diff = x[i] - scale_is * (float)l;
            mse += qw[i] * diff * diff;
        }
        if (mse < best_mse) { best_mse = mse; iscale = iscale_is; }
    }
    float sumlx = 0, suml2 = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const int l = imin(nmax, nearest_int(iscale * x[i]));
        L[i] = l & 0xFF;
        sumlx += qw[i] * x[i] * (float)l;
        suml2 += qw[i] * (float)l * (float)l;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float w = qw[i];
            const float li = (float)L[i];
            float slx = sumlx - w * x[i] * li;
            float sl2 = suml2 - w * li * li;
            if (slx > 0 && sl2 > 0) {
                const int new_l = imin(nmax, nearest_int(x[i] * sl2 / slx));
                if (new_l != L[i]) {
                    slx += w * x[i] * (float)new_l;
                    sl2 += w * (float)new_l * (float)new_l;
                    if (slx * slx * suml2 > sumlx * sumlx * sl2) {
                        L[i] = new_l & 0xFF;
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

// Best of the precomputed neighbours of an off-codebook lattice point: first strict minimum of
// sum_i w[i] * (scale*q[i] - x[i])^2 with the terms added in coordinate order.  Writes the
// winner's levels to L[0..GD) and returns its codebook index.
template <int GD>
GGUF_D int best_neighbour(const uint16_t *__restrict__ nb, const float *gridf, const float *xv, const float *wv, float scale,
                          int *L) {
    const int n = __ldg(nb);
    float best_d2 = FLT_MAX;
    int best = -1;
    int g_next = __ldg(nb + 1);  // the index of the next entry is fetched while the current one is evaluated
    for (int j = 1; j <= n; ++j) {
        const int g = g_next;
        g_next = __ldg(nb + (j < n ? j + 1 : j));
        float q[GD];
#pragma unroll
        for (int v = 0; v < GD / 4; ++v) {
            const float4 t = *reinterpret_cast<const float4 *>(gridf + g * GD + 4 * v);
            q[4 * v] = t.x; q[4 * v + 1] = t.y; q[4 * v + 2] = t.z; q[4 * v + 3] = t.w;
        }
        float d2 = 0;
#pragma unroll
        for (int i = 0; i < GD; ++i) {
            const float diff = scale * q[i] - xv[i];
            d2 += wv[i] * diff * diff;
        }
        if (d2 < best_d2) { best_d2 = d2; best = g; }
    }
#pragma unroll
    for (int v = 0; v < GD / 4; ++v) {
        const float4 t = *reinterpret_cast<const float4 *>(gridf + best * GD + 4 * v);
        // coordinates are 2*level + 1
        L[4 * v] = ((int)t.x - 1) >> 1; L[4 * v + 1] = ((int)t.y - 1) >> 1; L[4 * v + 2] = ((int)t.z - 1) >> 1; L[4 * v + 3] = ((int)t.w - 1) >> 1;
    }
    return best;
}

template <int TYPE>
__global__ void __launch_bounds__(kThreads) quant_iq23_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                             uint8_t *__restrict__ dst, int64_t nblocks, int64_t n_per_row,
                                                             IqSearchTable tab) {
    using T = Traits<TYPE>;
    constexpr int BS = T::BS, GD = T::GD, NG = BS / GD, NS = BS / 8, W = 256 / BS;  // W lanes per super-block
    // the codebook's coordinates as floats: no conversion in the neighbour scans, one or two 16-byte reads per entry
    extern __shared__ __align__(16) float gridf[];
    for (int i = threadIdx.x; i < tab.grid_size * GD; i += kThreads) gridf[i] = (float)__ldg(tab.grid + i);
    __syncthreads();

    const int lane = threadIdx.x & 31, j = lane & (W - 1), gbase = lane & ~(W - 1);
    int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = blk < nblocks;
    if (!active) blk = nblocks - 1;
    float xb[BS];
    load_group<BS>(src + blk * BS, xb);

    // sum of squares over the super-block, in element order (lane to lane)
    float sumx2 = 0.f;
#pragma unroll 1
    for (int s = 0; s < W; ++s) {
        if (j == s) {
#pragma unroll
            for (int i = 0; i < BS; ++i) sumx2 += xb[i] * xb[i];
        }
        sumx2 = __shfl_sync(kFull, sumx2, gbase + s);
    }
    const float sigma2 = T::SIGMA_X2 ? 2 * sumx2 / QK_K : sumx2 / QK_K;

    float weight[BS], waux[BS], xval[BS];
    if (qw) {
        const float *qwp = qw + (blk * BS) % n_per_row;
#pragma unroll
        for (int i = 0; i < BS; ++i) weight[i] = __ldg(qwp + i) * sqrtf(sigma2 + xb[i] * xb[i]);
    } else {
#pragma unroll
        for (int i = 0; i < BS; ++i) weight[i] = TYPE == GGML_TYPE_IQ2_S ? 0.25f * sigma2 + xb[i] * xb[i] : xb[i] * xb[i];
    }
#pragma unroll
    for (int i = 0; i < BS; ++i) waux[i] = sqrtf(weight[i]);

    uint32_t signs[NS];
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        uint32_t s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (xb[8 * k + i] >= 0) xval[8 * k + i] = xb[8 * k + i];
            else { xval[8 * k + i] = -xb[8 * k + i]; s |= 1u << i; }
        }
        if (T::PARITY) {
            if (__popc(s) & 1) {
                int im = 0;
                float mn = weight[8 * k] * xb[8 * k] * xb[8 * k];
#pragma unroll
                for (int i = 1; i < 8; ++i) {
                    const float ax = weight[8 * k + i] * xb[8 * k + i] * xb[8 * k + i];
                    if (ax < mn) { mn = ax; im = i; }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) if (i == im) xval[8 * k + i] = -xval[8 * k + i];
                s ^= 1u << im;
            }
            s &= 127;
        }
        signs[k] = s;
    }
    float max = xval[0];
#pragma unroll
    for (int i = 1; i < BS; ++i) max = max > xval[i] ? max : xval[i];

    uint32_t L[BS / 4];
#pragma unroll
    for (int i = 0; i < BS / 4; ++i) L[i] = 0;
    float scale = 0.f;
    bool skipped = T::EPS > 0.f ? (max < T::EPS) : !(max != 0.f);
    float eff_max = max;
    if (!skipped && T::QP_INIT) {
        int Linit[BS];
        scale = qp_quants_reg<BS>(T::KMAXQ + 1, xval, Linit, weight);
        eff_max = scale * T::KMAXQ;
        if (eff_max <= 0) {
            skipped = true;
            scale = 0.f;
        } else {
#pragma unroll
            for (int i = 0; i < BS; ++i) lset(L, i, Linit[i]);
        }
    }
    int gidx[NG];
#pragma unroll
    for (int k = 0; k < NG; ++k) gidx[k] = 0;

    if (!skipped) {
        float best = 0;
        if (!T::QP_INIT) scale = max / (2 * T::KMAXQ - 1);
        uint32_t on_grid = TYPE == GGML_TYPE_IQ3_S ? 0u : 0xFFFFFFFFu;  // bit k: group k of the accepted candidate was a codebook point
        // candidate by candidate, a neighbour scan wherever the rounding leaves the codebook
        for (int is = -T::IS_MAX; is <= T::IS_MAX; ++is) {
            const float id = ((float)(2 * T::KMAXQ - 1) + (float)is * T::STEP) / eff_max;
            const float this_scale = 1 / id;
            uint32_t Laux[BS / 4];
            uint32_t on_aux = 0;
            // the block's sums run over the elements in order, i.e. group by group: each group adds its terms as
            // soon as its levels are known
            float sumqx = 0, sumq2 = 0;
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                uint32_t u = 0;
                int lk[GD];
#pragma unroll
                for (int i = 0; i < GD; ++i) {
                    const int l = nearest_int(0.5f * (id * xval[GD * k + i] - 1));
                    lk[i] = imax(0, imin(T::KMAXQ - 1, l));
                    u |= (uint32_t)lk[i] << (T::BITS * i);
                }
                const int m = __ldg(tab.map + u);
                if (m < 0) best_neighbour<GD>(tab.neighbours + (-m - 1), gridf, xval + GD * k, waux + GD * k, this_scale, lk);
                else on_aux |= 1u << k;
#pragma unroll
                for (int i = 0; i < GD; ++i) {
                    const float w = weight[GD * k + i];
                    const float q = (float)(2 * lk[i] + 1);
                    sumqx += w * xval[GD * k + i] * q;
                    sumq2 += w * q * q;
                }
#pragma unroll
                for (int v = 0; v < GD / 4; ++v)
                    Laux[(GD * k) / 4 + v] = (uint32_t)lk[4 * v] | ((uint32_t)lk[4 * v + 1] << 8) | ((uint32_t)lk[4 * v + 2] << 16) | ((uint32_t)lk[4 * v + 3] << 24);
            }
            if (sumq2 > 0 && sumqx * sumqx > best * sumq2) {
                scale = sumqx / sumq2;
                best = scale * sumqx;
#pragma unroll
                for (int i = 0; i < BS / 4; ++i) L[i] = Laux[i];
                on_grid = on_aux;
            }
        }
        // re-projection at the accepted scale
        bool reproject;
        if (TYPE == GGML_TYPE_IQ2_XXS) reproject = scale > 0;
        else reproject = (on_grid & ((NG == 32) ? 0xFFFFFFFFu : ((1u << NG) - 1))) != ((NG == 32) ? 0xFFFFFFFFu : ((1u << NG) - 1)) && scale > 0;
        if (reproject) {
            const float id = 1 / scale;
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                const bool all_groups = TYPE == GGML_TYPE_IQ2_XXS || TYPE == GGML_TYPE_IQ3_S;
                if (!all_groups && ((on_grid >> k) & 1)) continue;
                uint32_t u = 0;
                int Lr[GD];
#pragma unroll
                for (int i = 0; i < GD; ++i) {
                    const int l = imax(0, imin(T::KMAXQ - 1, nearest_int(0.5f * (id * xval[GD * k + i] - 1))));
                    u |= (uint32_t)l << (T::BITS * i);
                    Lr[i] = l;
                }
                const int m = __ldg(tab.map + u);
                if (TYPE == GGML_TYPE_IQ2_XS || TYPE == GGML_TYPE_IQ2_S) {
                    // levels become the rounding, or the best neighbour when the rounding is off the codebook
                    if (m < 0) best_neighbour<GD>(tab.neighbours + (-m - 1), gridf, xval + GD * k, waux + GD * k, scale, Lr);
#pragma unroll
                    for (int i = 0; i < GD; ++i) lset(L, GD * k + i, Lr[i]);
                } else {
                    int g = m;
                    if (m < 0) g = best_neighbour<GD>(tab.neighbours + (-m - 1), gridf, xval + GD * k, waux + GD * k, scale, Lr);
#pragma unroll
                    for (int i = 0; i < GD; ++i) lset(L, GD * k + i, ((int)gridf[g * GD + i] - 1) >> 1);
                }
            }
            float sumqx = 0, sumq2 = 0;
#pragma unroll
            for (int i = 0; i < BS; ++i) {
                const float w = weight[i];
                const float q = (float)(2 * lget(L, i) + 1);
                sumqx += w * xval[i] * q;
                sumq2 += w * q * q;
            }
            if (sumq2 > 0) scale = sumqx / sumq2;
        }
        if (scale < 0) {
            scale = -scale;
            // upstream flips the first four sign bytes (all of them for the 16-element formats)
#pragma unroll
            for (int k = 0; k < NS; ++k) signs[k] = T::PARITY ? (~signs[k]) & 127 : (~signs[k]) & 0xFF;
        }
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            uint32_t u = 0;
#pragma unroll
            for (int i = 0; i < GD; ++i) u |= (uint32_t)lget(L, GD * k + i) << (T::BITS * i);
            const int m = __ldg(tab.map + u);
            gidx[k] = m < 0 ? 0 : m;  // upstream aborts here; every path above ends on a codebook point
        }
    }

    // ---- super-block stage ----
    float max_scale = skipped ? 0.f : scale;
#pragma unroll
    for (int m = 1; m < W; m <<= 1) {
        const float o = __shfl_xor_sync(kFull, max_scale, m);
        max_scale = max_scale > o ? max_scale : o;
    }
    const bool empty = !(max_scale != 0.f);
    const float d = max_scale / 31;
    const float idd = 1 / d;
    int lsc = 0;
    if (!empty) lsc = imax(0, imin(15, nearest_int(0.5f * (idd * (skipped ? 0.f : scale) - 1))));
    const int lsc_next = __shfl_down_sync(kFull, lsc, 1);
    // position of this block's payload for the format whose writer does not advance over skipped blocks
    const unsigned group_mask = (W == 32) ? kFull : (((1u << W) - 1) << gbase);
    const unsigned live = __ballot_sync(kFull, !skipped) & group_mask;
    const int nlive = __popc(live);
    const int rank_live = __popc(live & ((1u << lane) - 1));
    const int rank_dead = (lane - gbase) - rank_live;
    // IQ2_S: two bits per group of eight go to qh[ib/2]; gather the neighbour lane's bits
    uint32_t hi_bits = 0;
    if (TYPE == GGML_TYPE_IQ2_S) hi_bits = (uint32_t)(gidx[0] >> 8) | ((uint32_t)(gidx[NG > 1 ? 1 : 0] >> 8) << 2);
    const uint32_t hi_next = __shfl_down_sync(kFull, hi_bits, 1);
    if (!active) return;

    uint8_t *out = dst + (blk / W) * T::BYTES;
    const bool clear_all = empty && (TYPE == GGML_TYPE_IQ2_XXS || TYPE == GGML_TYPE_IQ2_XS || TYPE == GGML_TYPE_IQ3_XXS);
    if (j == 0) {
        float dd = d;
        if (TYPE == GGML_TYPE_IQ2_S) dd = d * 0.9875f;
        if (TYPE == GGML_TYPE_IQ3_XXS) dd = d * 1.0125f;
        if (TYPE == GGML_TYPE_IQ3_S) dd = d * 1.033f;
        st16(out, empty ? 0u : f32_to_half_bits(dd));
    }
    if constexpr (TYPE == GGML_TYPE_IQ2_XXS) {
        uint32_t w0 = 0, w1 = 0;
        if (!skipped && !clear_all) {
            w0 = (uint32_t)gidx[0] | ((uint32_t)gidx[1] << 8) | ((uint32_t)gidx[2] << 16) | ((uint32_t)gidx[3] << 24);
            w1 = signs[0] | (signs[1] << 7) | (signs[2] << 14) | (signs[3] << 21);
        }
        if (!clear_all) w1 |= (uint32_t)lsc << 28;
        st32(out + 2 + 8 * j, w0);
        st32(out + 2 + 8 * j + 4, w1);
    } else if constexpr (TYPE == GGML_TYPE_IQ2_XS) {
        uint32_t q0 = 0, q1 = 0;
        if (!skipped && !clear_all) { q0 = (uint32_t)gidx[0] | (signs[0] << 9); q1 = (uint32_t)gidx[1] | (signs[1] << 9); }
        st16(out + 2 + 4 * j, q0);
        st16(out + 2 + 4 * j + 2, q1);
        if ((j & 1) == 0) out[66 + (j >> 1)] = clear_all ? 0 : (uint8_t)(lsc | (lsc_next << 4));
    } else if constexpr (TYPE == GGML_TYPE_IQ2_S) {
        out[2 + 2 * j] = skipped ? 0 : (uint8_t)gidx[0];
        out[2 + 2 * j + 1] = skipped ? 0 : (uint8_t)gidx[1];
        out[2 + 32 + 2 * j] = skipped ? 0 : (uint8_t)signs[0];
        out[2 + 32 + 2 * j + 1] = skipped ? 0 : (uint8_t)signs[1];
        if ((j & 1) == 0) {
            out[66 + (j >> 1)] = (uint8_t)(hi_bits | (hi_next << 4));
            out[74 + (j >> 1)] = empty ? 0 : (uint8_t)(lsc | (lsc_next << 4));
        }
    } else if constexpr (TYPE == GGML_TYPE_IQ3_XXS) {
        uint32_t sas = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) out[2 + 8 * j + k] = (skipped || clear_all) ? 0 : (uint8_t)gidx[k];
        if (!skipped && !clear_all) sas = signs[0] | (signs[1] << 7) | (signs[2] << 14) | (signs[3] << 21);
        if (!clear_all) sas |= (uint32_t)lsc << 28;
        st32(out + 2 + 64 + 4 * j, sas);
    } else {  // IQ3_S: payload slots are consumed only by blocks that were not skipped
        const int pos = skipped ? nlive + rank_dead : rank_live;
        uint32_t qh = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            out[2 + 8 * pos + k] = skipped ? 0 : (uint8_t)gidx[k];
            qh |= (uint32_t)(gidx[k] >> 8) << k;
        }
        out[66 + j] = skipped ? 0 : (uint8_t)qh;
#pragma unroll
        for (int k = 0; k < 4; ++k) out[74 + 4 * pos + k] = skipped ? 0 : (uint8_t)signs[k];
        if ((j & 1) == 0) out[106 + (j >> 1)] = empty ? 0 : (uint8_t)(lsc | (lsc_next << 4));
    }
}

template <int TYPE>
cudaError_t launch(const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row, const DeviceState *state,
                   cudaStream_t stream) {
    using T = Traits<TYPE>;
    const IqSearchTable &tab = state->iq[T::TABLE];
    if (!tab.grid) return cudaErrorInvalidValue;
    const int64_t nblocks = nelems / T::BS;
    if (nblocks <= 0) return cudaSuccess;
    const size_t smem = (size_t)tab.grid_size * T::GD * sizeof(float);  // at most 32 KB
    const int64_t grid = (nblocks + kThreads - 1) / kThreads;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    quant_iq23_kernel<TYPE><<<(unsigned)grid, kThreads, smem, stream>>>(src, qw, static_cast<uint8_t *>(dst), nblocks, n_per_row, tab);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_quantize_iq1(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                                const DeviceState *state, cudaStream_t stream);

cudaError_t launch_quantize_iq(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                               const DeviceState *state, cudaStream_t stream) {
    if (!state) return cudaErrorInvalidValue;
    switch (type) {
        case GGML_TYPE_IQ2_XXS: return launch<GGML_TYPE_IQ2_XXS>(src, qw, dst, nelems, n_per_row, state, stream);
        case GGML_TYPE_IQ2_XS: return launch<GGML_TYPE_IQ2_XS>(src, qw, dst, nelems, n_per_row, state, stream);
        case GGML_TYPE_IQ2_S: return launch<GGML_TYPE_IQ2_S>(src, qw, dst, nelems, n_per_row, state, stream);
        case GGML_TYPE_IQ3_XXS: return launch<GGML_TYPE_IQ3_XXS>(src, qw, dst, nelems, n_per_row, state, stream);
        case GGML_TYPE_IQ3_S: return launch<GGML_TYPE_IQ3_S>(src, qw, dst, nelems, n_per_row, state, stream);
        case GGML_TYPE_IQ1_S: case GGML_TYPE_IQ1_M:
            return launch_quantize_iq1(type, src, qw, dst, nelems, n_per_row, state, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gguf
