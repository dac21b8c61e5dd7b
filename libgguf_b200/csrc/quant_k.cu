// K-quant quantizers Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, with and without importance weights.
//
// Mapping: one thread per sub-block (32 elements for Q4_K/Q5_K, 16 for Q2_K/Q3_K/Q6_K), the 8 or
// 16 threads of a super-block adjacent in a warp.  The sub-block search is the sequential upstream
// search run from registers (search.cuh); the super-block stage (largest scale, 6/4-bit scale
// codes, fp16 super-scales) is done with shuffles inside the 8- or 16-lane group because it only
// needs order-free maxima; the bit packing gathers the partner lanes' levels with shuffles.
// These kernels are bound by the fp32 pipe (several hundred dependent-free flops per element), not
// by memory, so input is read with plain 16-byte loads and output written in small pieces.
#include <math.h>

#include "gguf_common.cuh"
#include "kernels.h"
#include "search.cuh"

namespace gguf {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kThreads = 128;

template <int W>
GGUF_D float group_max(float v) {
#pragma unroll
    for (int m = 1; m < W; m <<= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, m));
    return v;
}

// Signed value with the largest magnitude among the W lanes of a group; on ties the lowest lane
// wins (upstream scans sub-blocks in order with a strict '>').
template <int W>
GGUF_D float group_first_absmax(float v, int lane_in_group) {
    float a = fabsf(v);
    int idx = lane_in_group;
#pragma unroll
    for (int m = 1; m < W; m <<= 1) {
        const float oa = __shfl_xor_sync(kFull, a, m);
        const float ov = __shfl_xor_sync(kFull, v, m);
        const int oi = __shfl_xor_sync(kFull, idx, m);
        if (oa > a || (oa == a && oi < idx)) { a = oa; v = ov; idx = oi; }
    }
    return v;
}

template <int N>
GGUF_D void load_group(const float *p, float (&x)[N]) {
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p) + k);
        x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
    }
}

GGUF_D void st16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
GGUF_D void st_word(uint8_t *p, uint32_t v) {
    p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); p[2] = (uint8_t)(v >> 16); p[3] = (uint8_t)(v >> 24);
}

// Sum of squares of the W*N elements of a super-block in element order: the partial sum is handed
// from lane to lane so the additions happen in exactly the upstream sequence.
template <int N, int W>
GGUF_D float group_ordered_sumsq(const float (&x)[N], int lane_in_group, int group_base_lane) {
    float acc = 0.f;
#pragma unroll 1
    for (int s = 0; s < W; ++s) {
        if (lane_in_group == s) {
#pragma unroll
            for (int i = 0; i < N; ++i) acc += x[i] * x[i];
        }
        acc = __shfl_sync(kFull, acc, group_base_lane + s);
    }
    return acc;
}

// per-warp scratch for the weighted variants' second-level search
struct WarpScratch {
    float scales[32];
    float mins[32];
    float sw[32];
    uint8_t Ls[32];
    uint8_t Lm[32];
    float dm[8];  // per super-block: d, dmin
};

// ---------------------------------------------------------------------------------------------
// Q4_K / Q5_K.  upstream q4_k.cpp:18-110 and :162-251, q5_k.cpp:18-124 and :187-301.
template <int NMAX, bool WEIGHTED>
__global__ void __launch_bounds__(kThreads) quant_q45k_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                             uint8_t *__restrict__ dst, int64_t n_sub, int64_t n_per_row) {
    constexpr int BYTES = NMAX == 15 ? 144 : 176;
    constexpr int QS_OFF = NMAX == 15 ? 16 : 48;
    __shared__ WarpScratch scratch[kThreads / 32];
    const int lane = threadIdx.x & 31, j = lane & 7, gbase = lane & ~7;
    int64_t sub = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = sub < n_sub;
    if (!active) sub = n_sub - 1;  // keep the warp convergent for the shuffles; results discarded
    const int64_t sb = sub >> 3;
    float x[32], w[32];
    load_group<32>(src + sub * 32, x);

    float scale, the_min;
    uint32_t L[8];
    uint32_t ls, lm;
    uint16_t d16, dmin16;
    if constexpr (!WEIGHTED) {
        float sum_x2 = 0;
#pragma unroll
        for (int l = 0; l < 32; ++l) sum_x2 += x[l] * x[l];
        const float av_x = sqrtf(sum_x2 / 32);
#pragma unroll
        for (int l = 0; l < 32; ++l) w[l] = av_x + fabsf(x[l]);
        if constexpr (NMAX == 15) scale = search_scale_min<32, false>(x, w, 15, -1.f, 0.1f, 20, the_min, L);
        else scale = search_scale_min<32, false>(x, w, 31, -0.5f, 0.1f, 15, the_min, L);
        const float max_scale = group_max<8>(fmaxf(scale, 0.f));
        const float max_min = group_max<8>(fmaxf(the_min, 0.f));
        const float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        const float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        ls = (uint32_t)nearest_int(inv_scale * scale) & 0xFF;
        lm = (uint32_t)nearest_int(inv_min * the_min) & 0xFF;
        ls = ls < 63 ? ls : 63;
        lm = lm < 63 ? lm : 63;
        d16 = f32_to_half_bits(max_scale / 63.f);
        dmin16 = f32_to_half_bits(max_min / 63.f);
    } else {
        const float sum_x2 = group_ordered_sumsq<32, 8>(x, j, gbase);
        const float sigma2 = 2 * sum_x2 / QK_K;
        const float *qwp = qw + (sub * 32) % n_per_row;
#pragma unroll
        for (int l = 0; l < 32; ++l) w[l] = __ldg(qwp + l) * sqrtf(sigma2 + x[l] * x[l]);
        float sumw = 0;
#pragma unroll
        for (int l = 0; l < 32; ++l) sumw += w[l];
        scale = search_scale_min<32, false>(x, w, NMAX, -0.9f, 0.05f, 36, the_min, L);
        WarpScratch &ws = scratch[threadIdx.x >> 5];
        ws.scales[lane] = scale;
        ws.mins[lane] = the_min;
        ws.sw[lane] = sumw;
        __syncwarp();
        if (j == 0) ws.dm[(gbase >> 3) * 2] = search_scale_positive(8, 63, ws.scales + gbase, ws.Ls + gbase, ws.sw + gbase);
        if (j == 1) ws.dm[(gbase >> 3) * 2 + 1] = search_scale_positive(8, 63, ws.mins + gbase, ws.Lm + gbase, ws.sw + gbase);
        __syncwarp();
        ls = ws.Ls[lane];
        lm = ws.Lm[lane];
        if (NMAX == 31) { ls = ls < 63 ? ls : 63; lm = lm < 63 ? lm : 63; }
        d16 = f32_to_half_bits(ws.dm[(gbase >> 3) * 2]);
        dmin16 = f32_to_half_bits(ws.dm[(gbase >> 3) * 2 + 1]);
        __syncwarp();
    }

    // The 6-bit codes survive the 12-byte packing unchanged, so requantize from them directly.
    const float d = half_bits_to_f32(d16) * (float)(ls & 63);
    if (d != 0.f) {
        const float dm = half_bits_to_f32(dmin16) * (float)(lm & 63);
        float lf[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) lf[i] = (float)imax(0, imin(NMAX, nearest_int((x[i] + dm) / d)));
        pack_levels<32>(lf, L);
    }

    uint8_t *out = dst + sb * BYTES;
    // scales[12]: lanes 0..3 own bytes j and j+4, lanes 4..7 own byte j+4.
    const uint32_t ls_p = __shfl_xor_sync(kFull, ls, 4);
    const uint32_t lm_p = __shfl_xor_sync(kFull, lm, 4);
    // high bits of this lane's levels, one bit per element (Q5_K)
    uint32_t hb = 0;
    if constexpr (NMAX == 31) {
#pragma unroll
        for (int i = 0; i < 32; ++i) hb |= (uint32_t)((level_at<32>(L, i) >> 4) & 1) << i;
    }
    // low nibbles of the partner lane (lane^1): pair (2g, 2g+1) shares the 32 qs bytes of 64-group g
    uint32_t Lp[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) Lp[k] = __shfl_xor_sync(kFull, L[k], 1);
    uint32_t hbs[8];
    if constexpr (NMAX == 31) {
#pragma unroll
        for (int s = 0; s < 8; ++s) hbs[s] = __shfl_sync(kFull, hb, gbase + s);
    }
    if (!active) return;
    if (j == 0) { st16(out, d16); st16(out + 2, dmin16); }
    if (j < 4) {
        out[4 + j] = (uint8_t)((ls & 63) | ((ls_p >> 4) << 6));
        out[8 + j] = (uint8_t)((lm & 63) | ((lm_p >> 4) << 6));
    } else {
        out[8 + j] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
    }
    if constexpr (NMAX == 31) {
        // qh[l] bit s = fifth bit of element l of sub-block s; lane j writes qh[4j .. 4j+3]
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int l = 4 * j + b;
            uint32_t byte = 0;
#pragma unroll
            for (int s = 0; s < 8; ++s) byte |= ((hbs[s] >> l) & 1) << s;
            out[16 + l] = (uint8_t)byte;
        }
    }
    // Even lane writes qs words 0..3 of its pair, odd lane words 4..7.
    uint8_t *qs = out + QS_OFF + 32 * (j >> 1);
    const int k0 = (j & 1) ? 4 : 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = (j & 1) ? Lp[k0 + k] : L[k0 + k];
        const uint32_t hi = (j & 1) ? L[k0 + k] : Lp[k0 + k];
        st_word(qs + 4 * (k0 + k), (lo & 0x0F0F0F0Fu) | ((hi & 0x0F0F0F0Fu) << 4));
    }
}

// ---------------------------------------------------------------------------------------------
// 2-bit plane packing shared by Q2_K and Q3_K: byte l of half h holds elements 128h + l + 32q,
// q = 0..3, i.e. lanes 8h + 2q + (l/16).  `two_bits` holds this lane's 16 levels, 2 bits each.
GGUF_D void store_2bit_planes(uint8_t *qs, uint32_t two_bits, int j, bool active) {
    const int h = j >> 3, p = j & 1;
    const int src0 = (threadIdx.x & 16) + 8 * h + p;
    const uint32_t t0 = __shfl_sync(kFull, two_bits, src0);
    const uint32_t t1 = __shfl_sync(kFull, two_bits, src0 + 2);
    const uint32_t t2 = __shfl_sync(kFull, two_bits, src0 + 4);
    const uint32_t t3 = __shfl_sync(kFull, two_bits, src0 + 6);
    // lanes with q == 0 write 8 bytes each of their (h, p) run: q-index of this lane selects the half
    const int q = (j >> 1) & 3;
    if (!active || q >= 2) return;
    uint8_t *o = qs + 32 * h + 16 * p + 8 * q;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = 8 * q + i;
        o[i] = (uint8_t)(((t0 >> (2 * e)) & 3) | (((t1 >> (2 * e)) & 3) << 2) | (((t2 >> (2 * e)) & 3) << 4) |
                         (((t3 >> (2 * e)) & 3) << 6));
    }
}

// Q2_K.  upstream q2_k.cpp:18-106 and :169-242.
template <bool WEIGHTED>
__global__ void __launch_bounds__(kThreads) quant_q2k_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                            uint8_t *__restrict__ dst, int64_t n_sub, int64_t n_per_row) {
    __shared__ WarpScratch scratch[kThreads / 32];
    const int lane = threadIdx.x & 31, j = lane & 15, gbase = lane & ~15;
    int64_t sub = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = sub < n_sub;
    if (!active) sub = n_sub - 1;
    const int64_t sb = sub >> 4;
    float x[16], w[16];
    load_group<16>(src + sub * 16, x);
    float scale, the_min;
    uint32_t L[4];
    uint32_t sc_byte;
    uint16_t d16, dmin16;
    if constexpr (!WEIGHTED) {
#pragma unroll
        for (int l = 0; l < 16; ++l) w[l] = fabsf(x[l]);
        scale = search_scale_min<16, true>(x, w, 3, -0.5f, 0.1f, 15, the_min, L);
        const float max_scale = group_max<16>(fmaxf(scale, 0.f));
        const float max_min = group_max<16>(fmaxf(the_min, 0.f));
        sc_byte = 0;
        d16 = f32_to_half_bits(0.f);
        dmin16 = f32_to_half_bits(0.f);
        if (max_scale > 0) {
            const float iscale = 15.f / max_scale;
            sc_byte = (uint32_t)nearest_int(iscale * scale) & 0xFF;
            d16 = f32_to_half_bits(max_scale / 15.f);
        }
        if (max_min > 0) {
            const float iscale = 15.f / max_min;
            sc_byte = (sc_byte | ((uint32_t)nearest_int(iscale * the_min) << 4)) & 0xFF;
            dmin16 = f32_to_half_bits(max_min / 15.f);
        }
    } else {
        const float sumx2 = group_ordered_sumsq<16, 16>(x, j, gbase);
        const float sigma2 = sumx2 / QK_K;
        const float *qwp = qw + (sub * 16) % n_per_row;
#pragma unroll
        for (int l = 0; l < 16; ++l) w[l] = __ldg(qwp + l) * sqrtf(sigma2 + x[l] * x[l]);
        float sumw = 0;
#pragma unroll
        for (int l = 0; l < 16; ++l) sumw += w[l];
        scale = search_scale_min<16, false>(x, w, 3, -0.9f, 0.05f, 36, the_min, L);
        WarpScratch &ws = scratch[threadIdx.x >> 5];
        ws.scales[lane] = scale;
        ws.mins[lane] = the_min;
        ws.sw[lane] = sumw;
        __syncwarp();
        if (j == 0) ws.dm[(gbase >> 4) * 2] = search_scale_positive(16, 15, ws.scales + gbase, ws.Ls + gbase, ws.sw + gbase);
        if (j == 1) ws.dm[(gbase >> 4) * 2 + 1] = search_scale_positive(16, 15, ws.mins + gbase, ws.Lm + gbase, ws.sw + gbase);
        __syncwarp();
        sc_byte = ((uint32_t)ws.Ls[lane] | ((uint32_t)ws.Lm[lane] << 4)) & 0xFF;
        d16 = f32_to_half_bits(ws.dm[(gbase >> 4) * 2]);
        dmin16 = f32_to_half_bits(ws.dm[(gbase >> 4) * 2 + 1]);
        __syncwarp();
    }
    const float d = half_bits_to_f32(d16) * (float)(sc_byte & 0xF);
    if (d != 0.f) {
        const float dm = half_bits_to_f32(dmin16) * (float)(sc_byte >> 4);
        float lf[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) lf[i] = (float)imax(0, imin(3, nearest_int((x[i] + dm) / d)));
        pack_levels<16>(lf, L);
    }
    uint32_t two_bits = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) two_bits |= (uint32_t)(level_at<16>(L, i) & 3) << (2 * i);
    uint8_t *out = dst + sb * 84;
    store_2bit_planes(out + 16, two_bits, j, active);
    if (!active) return;
    out[j] = (uint8_t)sc_byte;
    if (j == 0) { st16(out + 80, d16); st16(out + 82, dmin16); }
}

// Q3_K.  upstream q3_k.cpp:18-113 and :176-280.
template <bool WEIGHTED>
__global__ void __launch_bounds__(kThreads) quant_q3k_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                            uint8_t *__restrict__ dst, int64_t n_sub, int64_t n_per_row) {
    const int lane = threadIdx.x & 31, j = lane & 15, gbase = lane & ~15;
    int64_t sub = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = sub < n_sub;
    if (!active) sub = n_sub - 1;
    const int64_t sb = sub >> 4;
    float x[16];
    load_group<16>(src + sub * 16, x);
    uint32_t L[4];
    int l6;  // 6-bit scale code, 0..63
    uint16_t d16;
    if constexpr (!WEIGHTED) {
        const float scale = search_scale_descent<16>(x, 4, L);
        const float max_scale = group_first_absmax<16>(scale, j);
        l6 = 0;
        d16 = f32_to_half_bits(0.f);
        if (max_scale != 0.f) {
            const float iscale = -32.f / max_scale;
            int l = (int)(int8_t)nearest_int(iscale * scale);
            l6 = imax(-32, imin(31, l)) + 32;
            d16 = f32_to_half_bits(1 / iscale);
        }
    } else {
        const float sumx2 = group_ordered_sumsq<16, 16>(x, j, gbase);
        const float sigma2 = 2 * sumx2 / QK_K;
        float w[16];
        const float *qwp = qw + (sub * 16) % n_per_row;
#pragma unroll
        for (int l = 0; l < 16; ++l) w[l] = __ldg(qwp + l) * sqrtf(sigma2 + x[l] * x[l]);
        float sumw = 0;
#pragma unroll
        for (int l = 0; l < 16; ++l) sumw += w[l];
        const float scale = search_scale_sym<16, true>(x, w, 4, L);
        // second level: every lane of the group runs the same 16-value search on the gathered scales
        float sc[16], sw[16];
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            sc[s] = __shfl_sync(kFull, scale, gbase + s);
            sw[s] = __shfl_sync(kFull, sumw, gbase + s);
        }
        uint32_t Ls[4];
        const float d_block = search_scale_sym<16, true>(sc, sw, 32, Ls);
        l6 = 0;
#pragma unroll
        for (int s = 0; s < 16; ++s) if (s == j) l6 = level_at<16>(Ls, s);
        d16 = f32_to_half_bits(d_block);
    }
    {
        const int sc = l6 - 32;
        const float d = half_bits_to_f32(d16) * (float)sc;
        if (d != 0.f) {
            float lf[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) lf[i] = (float)(imax(-4, imin(3, nearest_int(x[i] / d))) + 4);
            pack_levels<16>(lf, L);
        }
    }
    // split into the high bit (hmask) and the low two bits
    uint32_t two_bits = 0, high = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        int l = level_at<16>(L, i);
        if (l > 3) { high |= 1u << i; l -= 4; }
        two_bits |= (uint32_t)(l & 3) << (2 * i);
    }
    uint8_t *out = dst + sb * 110;
    store_2bit_planes(out + 32, two_bits, j, active);
    // hmask[m] bit (e/32) for element e = 16*s + i: m = e % 32 = 16*(s&1) + i, bit = s >> 1.
    // Lane j writes hmask bytes [2j, 2j+1]: m = 2j + b -> parity (2j+b)/16, i = (2j+b) % 16.
    uint32_t hs[16];
#pragma unroll
    for (int s = 0; s < 16; ++s) hs[s] = __shfl_sync(kFull, high, gbase + s);
    // scale codes: byte k<8 = low nibbles of codes k and k+8; byte 8+k (k<4) = top 2 bits of codes k, k+4, k+8, k+12
    int codes[16];
#pragma unroll
    for (int s = 0; s < 16; ++s) codes[s] = __shfl_sync(kFull, l6, gbase + s);
    if (!active) return;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        const int m = 2 * j + b, par = m >> 4, i = m & 15;
        uint32_t byte = 0;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
            uint32_t hv = 0;
#pragma unroll
            for (int s = 0; s < 16; ++s) if (s == 2 * s2 + par) hv = hs[s];
            byte |= ((hv >> i) & 1) << s2;
        }
        out[m] = (uint8_t)byte;
    }
    if (j < 8) {
        int lo = 0, hi = 0;
#pragma unroll
        for (int s = 0; s < 16; ++s) { if (s == j) lo = codes[s]; if (s == j + 8) hi = codes[s]; }
        out[96 + j] = (uint8_t)((lo & 0xF) | ((hi & 0xF) << 4));
    } else if (j < 12) {
        const int k = j - 8;
        int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            if (s == k) c0 = codes[s];
            if (s == k + 4) c1 = codes[s];
            if (s == k + 8) c2 = codes[s];
            if (s == k + 12) c3 = codes[s];
        }
        out[96 + 8 + k] = (uint8_t)((c0 >> 4) | ((c1 >> 4) << 2) | ((c2 >> 4) << 4) | ((c3 >> 4) << 6));
    } else if (j == 12) {
        st16(out + 108, d16);
    }
}

// Q6_K.  upstream q6_k.cpp:18-96 and :159-253.
template <bool WEIGHTED>
__global__ void __launch_bounds__(kThreads) quant_q6k_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                            uint8_t *__restrict__ dst, int64_t n_sub, int64_t n_per_row) {
    const int lane = threadIdx.x & 31, j = lane & 15;
    int64_t sub = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = sub < n_sub;
    if (!active) sub = n_sub - 1;
    const int64_t sb = sub >> 4;
    float x[16], w[16];
    load_group<16>(src + sub * 16, x);
    uint32_t L[4];
    float scale;
    if constexpr (WEIGHTED) {
        const float *qwp = qw + (sub * 16) % n_per_row;
#pragma unroll
        for (int l = 0; l < 16; ++l) w[l] = __ldg(qwp + l);
        scale = search_scale_sym<16, true>(x, w, 32, L);
    } else {
        scale = search_scale_sym<16, false>(x, w, 32, L);
    }
    const float max_scale = group_first_absmax<16>(scale, j);
    const bool empty = fabsf(max_scale) < 1e-15f;
    uint16_t d16 = 0;
    int sc8 = 0;
    if (!empty) {
        const float iscale = -128.f / max_scale;
        d16 = f32_to_half_bits(1 / iscale);
        sc8 = (int)(int8_t)imin(127, nearest_int(iscale * scale));
        const float d = half_bits_to_f32(d16) * (float)sc8;
        if (d != 0.f) {
            float lf[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) lf[i] = (float)(imax(-32, imin(31, nearest_int(x[i] / d))) + 32);
            pack_levels<16>(lf, L);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) L[k] = 0;
    }
    // Element 128h + 32q + 16p + i lives in lane 8h + 2q + p.  Lanes with q == 0 gather the other
    // three planes and write ql[64h + 16p + i], ql[64h + 32 + 16p + i] and qh[32h + 16p + i].
    const int h = j >> 3, p = j & 1;
    const int src0 = (lane & 16) + 8 * h + p;
    uint32_t P[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int k = 0; k < 4; ++k) P[q][k] = __shfl_sync(kFull, L[k], src0 + 2 * q);
    if (!active) return;
    uint8_t *out = dst + sb * 210;
    out[192 + j] = (uint8_t)(int8_t)sc8;
    if (j == 0) st16(out + 208, d16);
    const int q = (j >> 1) & 3;
    // spread the writing: lane q of the run writes word q of each of the three 16-byte pieces
    const uint32_t m0F = 0x0F0F0F0Fu, m03 = 0x03030303u;
    uint32_t ql_lo = 0, ql_hi = 0, qh_w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (k == q) {
            ql_lo = (P[0][k] & m0F) | ((P[2][k] & m0F) << 4);
            ql_hi = (P[1][k] & m0F) | ((P[3][k] & m0F) << 4);
            qh_w = ((P[0][k] >> 4) & m03) | (((P[1][k] >> 4) & m03) << 2) | (((P[2][k] >> 4) & m03) << 4) |
                   (((P[3][k] >> 4) & m03) << 6);
        }
    }
    st_word(out + 64 * h + 16 * p + 4 * q, ql_lo);
    st_word(out + 64 * h + 32 + 16 * p + 4 * q, ql_hi);
    st_word(out + 128 + 32 * h + 16 * p + 4 * q, qh_w);
}

template <class Kernel>
cudaError_t launch_sub(Kernel kernel, const float *src, const float *qw, void *dst, int64_t n_sub, int64_t n_per_row,
                       cudaStream_t stream) {
    if (n_sub <= 0) return cudaSuccess;
    const int64_t grid = (n_sub + kThreads - 1) / kThreads;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    kernel<<<(unsigned)grid, kThreads, 0, stream>>>(src, qw, static_cast<uint8_t *>(dst), n_sub, n_per_row);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_quantize_k(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                              cudaStream_t stream) {
    switch (type) {
        case GGML_TYPE_Q4_K:
            return qw ? launch_sub(quant_q45k_kernel<15, true>, src, qw, dst, nelems / 32, n_per_row, stream)
                      : launch_sub(quant_q45k_kernel<15, false>, src, qw, dst, nelems / 32, n_per_row, stream);
        case GGML_TYPE_Q5_K:
            return qw ? launch_sub(quant_q45k_kernel<31, true>, src, qw, dst, nelems / 32, n_per_row, stream)
                      : launch_sub(quant_q45k_kernel<31, false>, src, qw, dst, nelems / 32, n_per_row, stream);
        case GGML_TYPE_Q2_K:
            return qw ? launch_sub(quant_q2k_kernel<true>, src, qw, dst, nelems / 16, n_per_row, stream)
                      : launch_sub(quant_q2k_kernel<false>, src, qw, dst, nelems / 16, n_per_row, stream);
        case GGML_TYPE_Q3_K:
            return qw ? launch_sub(quant_q3k_kernel<true>, src, qw, dst, nelems / 16, n_per_row, stream)
                      : launch_sub(quant_q3k_kernel<false>, src, qw, dst, nelems / 16, n_per_row, stream);
        case GGML_TYPE_Q6_K:
            return qw ? launch_sub(quant_q6k_kernel<true>, src, qw, dst, nelems / 16, n_per_row, stream)
                      : launch_sub(quant_q6k_kernel<false>, src, qw, dst, nelems / 16, n_per_row, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gguf
