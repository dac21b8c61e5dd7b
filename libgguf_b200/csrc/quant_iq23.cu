// Lattice quantizers IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S.
//
// One lane owns 32 (IQ2_XXS) or 16 elements: a whole block, or for the IQ3 types half of a 32-element block (the
// two lanes of a block sit next to each other and hand the ordered sums from one to the other, which keeps the
// kernel at 96 registers and 19-20 warps per SM); the lanes of a super-block sit next to each other in a warp.
// Per block the upstream algorithm is run literally: sign extraction (with the even-parity fix where the format
// stores 7 sign bits), a loop over candidate scales in which every group of 8 (or 4) magnitudes is rounded to the
// lattice and, when the rounded point is not a codebook entry, replaced by the best of its precomputed neighbours,
// the accept/reject chain on (sumqx, sumq2), the final re-projection (run as one more pass of the same loop), and
// the 4-bit block scale against the super-block maximum.
//
// The neighbour scans are most of the arithmetic and their lengths differ from group to group (1 to about 300
// entries), so a lane that scanned its own lists left two thirds of the warp idle.  Here the warp works in rounds:
// every lane rounds its groups for one candidate and queues the scans that came up, the warp lays the queued lists
// end to end and every lane evaluates an equal stretch of that sequence (whatever lists it crosses), and the owners
// read the winners back and run the accept/reject chain.  The lists are kept in a layout of their own (whole,
// aligned records of four or eight entries, an entry being the offset of its codebook row), the codebook is staged
// in shared memory as bfloat16 pairs (exact for its small odd integers), every lane's magnitudes and root weights
// in padded rows.  The IQ3 codebooks' records (47 and 58 KB) are staged in shared memory too, under one CTA per SM
// that stays for the whole launch; of the IQ2_XS and IQ2_S records (1.1 and 0.5 MB) the front of the array, which
// holds the most common lattice points' lists, is staged the same way (84 and 76 KB) and the rest read from global
// memory; the IQ2_XXS records and every lattice map stay in global memory (L2).
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

template <int TYPE> struct Traits;
template <> struct Traits<GGML_TYPE_IQ2_XXS> {
    static constexpr int BS = 32, GD = 8, BITS = 2, KMAXQ = 3, IS_MAX = 6, BYTES = 66, TABLE = IQT_2XXS, THREADS = 128, CTAS = 4, REC = 1, LPB = 1;
    static constexpr bool LISTS_SHARED = false, LISTS_HOT = false, MERGED = true;
    static constexpr bool PARITY = true, SIGMA_X2 = false, QP_INIT = true;
    static constexpr float STEP = 0.1f, EPS = 1e-15f;
};
template <> struct Traits<GGML_TYPE_IQ2_XS> {
    static constexpr int BS = 16, GD = 8, BITS = 2, KMAXQ = 3, IS_MAX = 9, BYTES = 74, TABLE = IQT_2XS, THREADS = 640, CTAS = 1, REC = 2, LPB = 1;
    static constexpr bool LISTS_SHARED = false, LISTS_HOT = true, MERGED = false;  // 8 KB codebook + 20 warps x 6.75 KB + 84 KB of records
    static constexpr bool PARITY = true, SIGMA_X2 = false, QP_INIT = false;
    static constexpr float STEP = 0.1f, EPS = 1e-15f;
};
template <> struct Traits<GGML_TYPE_IQ2_S> {
    static constexpr int BS = 16, GD = 8, BITS = 2, KMAXQ = 3, IS_MAX = 9, BYTES = 82, TABLE = IQT_2S, THREADS = 640, CTAS = 1, REC = 1, LPB = 1;
    static constexpr bool LISTS_SHARED = false, LISTS_HOT = true, MERGED = false;  // 16 KB codebook + 20 warps x 6.75 KB + 76 KB of records
    static constexpr bool PARITY = false, SIGMA_X2 = true, QP_INIT = false;
    static constexpr float STEP = 0.1f, EPS = 1e-8f;
};
template <> struct Traits<GGML_TYPE_IQ3_XXS> {
    static constexpr int BS = 32, GD = 4, BITS = 3, KMAXQ = 8, IS_MAX = 15, BYTES = 98, TABLE = IQT_3XXS, THREADS = 640, CTAS = 1, REC = 1, LPB = 2;
    static constexpr bool MERGED = true, LISTS_SHARED = true, LISTS_HOT = false;  // 47 KB of records + 2 KB codebook + 20 warps x 8.5 KB
    static constexpr bool PARITY = true, SIGMA_X2 = true, QP_INIT = false;
    static constexpr float STEP = 0.2f, EPS = 1e-8f;
};
template <> struct Traits<GGML_TYPE_IQ3_S> {
    static constexpr int BS = 32, GD = 4, BITS = 3, KMAXQ = 8, IS_MAX = 9, BYTES = 110, TABLE = IQT_3S, THREADS = 608, CTAS = 1, REC = 1, LPB = 2;
    static constexpr bool MERGED = true, LISTS_SHARED = true, LISTS_HOT = false;  // 58 KB of records + 4 KB codebook + 19 warps x 8.5 KB
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

// Codebook row at byte offset `at` of the staged codebook: coordinates are small odd integers, kept as bfloat16 pairs
// (exact), so a row is one 16-byte (8 coordinates) or 8-byte (4 coordinates) read and a shift or mask per coordinate.
// As floats a row of eight took two 16-byte reads that used half of the banks, and the gathers of 32 lanes at 32
// random rows kept the shared-memory pipe busier than the arithmetic.
template <int GD>
GGUF_D void grid_row(const uint32_t *gridh, uint32_t at, float (&q)[GD]) {
    uint32_t w[GD / 2];
    const char *row = reinterpret_cast<const char *>(gridh) + at;
    if constexpr (GD == 8) {
        const uint4 t = *reinterpret_cast<const uint4 *>(row);
        w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    } else {
        const uint2 t = *reinterpret_cast<const uint2 *>(row);
        w[0] = t.x; w[1] = t.y;
    }
#pragma unroll
    for (int i = 0; i < GD / 2; ++i) {
        q[2 * i] = __uint_as_float(w[i] << 16);
        q[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
template <int GD>
GGUF_D void grid_entry(const uint32_t *gridh, int g, float (&q)[GD]) { grid_row<GD>(gridh, (uint32_t)g * (GD * 2), q); }

// Weighted squared distance of the codebook row at byte offset `at` from the group, terms added in coordinate order.
// nx holds the negated magnitudes (a - b is a + (-b) exactly).  Coordinates 2i and 2i+1 share two-wide instructions
// for the difference and its two multiplications; the products scale * q stay scalar multiplies (a packed multiply
// feeding a packed add would be contracted into a fused multiply-add) and the sum stays a chain of scalar adds.
template <int GD>
GGUF_D float neighbour_d2(const uint32_t *gridh, uint32_t at, float scale, const float2 (&nx)[GD / 2], const float2 (&wv)[GD / 2]) {
    float q[GD];
    grid_row<GD>(gridh, at, q);
    float d2 = 0;
#pragma unroll
    for (int i = 0; i < GD / 2; ++i) {
        const float2 diff = __fadd2_rn(make_float2(__fmul_rn(scale, q[2 * i]), __fmul_rn(scale, q[2 * i + 1])), nx[i]);
        const float2 term = __fmul2_rn(__fmul2_rn(wv[i], diff), diff);
        d2 = __fadd_rn(d2, term.x);
        d2 = __fadd_rn(d2, term.y);
    }
    return d2;
}

// a group's negated magnitudes / its root weights from the staged rows, as pairs
template <int GD>
GGUF_D void load_pairs(const float *p, float2 (&v)[GD / 2], bool negate) {
#pragma unroll
    for (int k = 0; k < GD / 4; ++k) {
        const float4 t = reinterpret_cast<const float4 *>(p)[k];
        v[2 * k] = negate ? make_float2(-t.x, -t.y) : make_float2(t.x, t.y);
        v[2 * k + 1] = negate ? make_float2(-t.z, -t.w) : make_float2(t.z, t.w);
    }
}

template <int N>
GGUF_D void load_staged(const float *p, float (&x)[N]) {  // shared memory, 16-byte aligned
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
        const float4 v = reinterpret_cast<const float4 *>(p)[k];
        x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
    }
}

// One neighbour scan a warp has to run: which list, which group of which lane's block, at which scale.
struct alignas(16) ScanTask {
    uint32_t base;   // the list's first record in the record array
    uint32_t nrec;   // its length in records
    float scale;
    uint32_t xoff;   // float offset of the group in the warp's staged magnitudes / weights
};

constexpr unsigned long long kNoWinner = ~0ull;
constexpr int PER = kIqStepEntries;
template <int REC> struct RecordOf;
template <> struct RecordOf<1> { using type = uint2; };
template <> struct RecordOf<2> { using type = uint4; };

// The warp's pending scans, evaluated with the work spread evenly.  A list is a whole number of records of REC steps
// of PER entries (its tail repeats its first entry, which can never be a strict improvement), so the T lists laid end
// to end are S records (`first[t]` = position of list t's first record) and every lane takes a contiguous stretch
// of S/32 records, whatever lists it crosses: every lane runs the same number of iterations, each one aligned 8- or
// 16-byte load and, per step, PER independent ordered sums with no bookkeeping per entry.  (32 lanes loading from 32
// different lines cost the L1 / shared-memory pipe as much as the steps' codebook gathers, which is why the long lists
// use two-step records.)  A list's winner is the first strict minimum in list order, i.e. the minimum of (distance
// bits, position) as one 64-bit key; a lane that saw a whole list stores its key, lanes that share a list combine
// theirs with a shared-memory atomic minimum.  Distances are sums of non-negative terms, so their bit patterns order
// like the floats; a NaN or FLT_MAX never wins, as upstream's `<` against FLT_MAX.
template <int GD, int TMAX, int REC, bool SHARED, bool HOT>
GGUF_D void balanced_scan(int lane, int T, uint32_t S, const ScanTask *tasks, const uint32_t *first, unsigned long long *winner,
                          const float *xs, const float *ws, const uint32_t *gridh, const void *__restrict__ records, uint32_t nhot = 0,
                          const void *__restrict__ cold_records = nullptr) {
    using Record = typename RecordOf<REC>::type;
    // records in global memory are fetched this many iterations early, across list boundaries; records in shared
    // memory are read where they are used (no second cursor to keep)
    constexpr int AHEAD = REC == 1 ? 3 : 2;
    const Record *const recs = static_cast<const Record *>(records);
    const uint32_t share = (S + 31) >> 5;
    uint32_t s = umin((uint32_t)lane * share, S);
    const uint32_t end = umin(s + share, S);
    if (s >= end) return;
    int t = 0;
#pragma unroll
    for (int step = TMAX / 2; step; step >>= 1) {
        const int c = t + step;
        if (c < T && first[c] <= s) t = c;
    }
    ScanTask tk = tasks[t];
    float2 xv[GD / 2], wv[GD / 2];
    load_pairs<GD>(xs + tk.xoff, xv, true);
    load_pairs<GD>(ws + tk.xoff, wv, false);
    uint32_t j = s - first[t];
    bool whole = j == 0;
    float best_d2 = FLT_MAX;
    uint32_t best_at = 0xFFFFFFFFu;
    // the fetch cursor runs AHEAD records in front of the evaluation cursor
    int ft = t;
    uint32_t fleft = tk.nrec - j, fs = s;
    const Record *fp = recs + tk.base + j;
    Record ring[AHEAD];
    auto fetch = [&](Record &rec) {
        if (!SHARED && !HOT && fs < end) {
            rec = __ldg(fp);
            ++fp;
            ++fs;
            if (--fleft == 0 && fs < end) {
                ++ft;
                const uint2 h = *reinterpret_cast<const uint2 *>(tasks + ft);
                fp = recs + h.x;
                fleft = h.y;
            }
        }
    };
#pragma unroll
    for (int d = 0; d < AHEAD; ++d) { ring[d] = Record(); fetch(ring[d]); }
    while (s < end) {
        Record rec;
        if constexpr (SHARED) {
            rec = recs[tk.base + j];
        } else if constexpr (HOT) {
            // the front of the record array (the most common lattice points' lists) is in shared memory, the rest in global
            const uint32_t at_record = tk.base + j;
            if (at_record < nhot) rec = recs[at_record];
            else rec = __ldg(static_cast<const Record *>(cold_records) + at_record);
        } else {
            rec = ring[0];
#pragma unroll
            for (int d = 0; d + 1 < AHEAD; ++d) ring[d] = ring[d + 1];
            fetch(ring[AHEAD - 1]);
        }
        static_assert(PER == 4, "a step is two words of two 16-bit row offsets");
        uint32_t words[2 * REC];
        if constexpr (REC == 1) { words[0] = rec.x; words[1] = rec.y; }
        else { words[0] = rec.x; words[1] = rec.y; words[2] = rec.z; words[3] = rec.w; }
#pragma unroll
        for (int h = 0; h < REC; ++h) {
            const uint32_t at[PER] = {words[2 * h] & 0xFFFFu, words[2 * h] >> 16, words[2 * h + 1] & 0xFFFFu, words[2 * h + 1] >> 16};
            float d2[PER];
#pragma unroll
            for (int q = 0; q < PER; ++q) d2[q] = neighbour_d2<GD>(gridh, at[q], tk.scale, xv, wv);
            const uint32_t pos = (j * REC + h) << 18;  // (entry position of the step) << 16
#pragma unroll
            for (int q = 0; q < PER; ++q) {
                if (d2[q] < best_d2) { best_d2 = d2[q]; best_at = pos + ((uint32_t)q << 16) + at[q]; }
            }
        }
        ++s;
        ++j;
        if (j == tk.nrec) {
            if (best_d2 < FLT_MAX) {
                const unsigned long long key = ((unsigned long long)__float_as_uint(best_d2) << 32) | best_at;
                if (whole) winner[t] = key;
                else atomicMin(winner + t, key);
            }
            ++t;
            j = 0;
            whole = true;
            best_d2 = FLT_MAX;
            best_at = 0xFFFFFFFFu;
            if (s < end) {
                tk = tasks[t];
                load_pairs<GD>(xs + tk.xoff, xv, true);
                load_pairs<GD>(ws + tk.xoff, wv, false);
            }
        }
    }
    if (j != 0 && best_d2 < FLT_MAX)
        atomicMin(winner + t, ((unsigned long long)__float_as_uint(best_d2) << 32) | best_at);
}

template <int TYPE>
__global__ void __launch_bounds__(Traits<TYPE>::THREADS, Traits<TYPE>::CTAS) quant_iq23_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                             uint8_t *__restrict__ dst, int64_t nlanes, int64_t n_per_row,
                                                             IqSearchTable tab) {
    using T = Traits<TYPE>;
    // A block of BS elements belongs to LPB neighbouring lanes, EL elements (NG groups) each; W lanes per super-block.
    constexpr int BS = T::BS, LPB = T::LPB, EL = BS / LPB, GD = T::GD, NG = EL / GD, NS = EL / 8, W = 256 / EL;
    static_assert(LPB == 1 || LPB == 2, "one or two lanes per block");
    static_assert(!(T::QP_INIT && LPB != 1), "the initial scale search runs over a whole block in one lane");
    constexpr int kThreads = T::THREADS;
    extern __shared__ __align__(16) uint32_t gridh[];
    for (int i = threadIdx.x; i < tab.grid_size * GD / 2; i += kThreads) {
        const uint32_t lo = __float_as_uint((float)__ldg(tab.grid + 2 * i)), hi = __float_as_uint((float)__ldg(tab.grid + 2 * i + 1));
        gridh[i] = (lo >> 16) | (hi & 0xFFFF0000u);
    }
    // The codebooks whose neighbour records fit (IQ3: 47 and 58 KB) keep them in shared memory next to the codebook,
    // one copy per SM under a CTA that stays for the whole launch: a step's record is then a shared-memory read of
    // a few wavefronts instead of a global load that touches 32 lines.
    const void *records = tab.records;
    int state_words = tab.grid_size * (GD / 2);
    if constexpr (T::LISTS_SHARED || T::LISTS_HOT) {
        uint2 *const staged = reinterpret_cast<uint2 *>(gridh + state_words);
        const uint2 *const from = static_cast<const uint2 *>(tab.records);
        const int staged_bytes = T::LISTS_SHARED ? tab.records_bytes : tab.hot_bytes;   // a multiple of 16
        for (int i = threadIdx.x; i < staged_bytes / 8; i += kThreads) staged[i] = __ldg(from + i);
        records = staged;
        // (rounded although it is whole already: the expression tells the compiler the alignment of what follows, and the
        // IQ3 kernels are 4 % slower without it)
        state_words += (staged_bytes / 4 + 3) & ~3;
    }
    __syncthreads();
    // per warp: every lane's magnitudes and root weights in rows padded by four floats, the pending
    // scans of one candidate, where each list starts in the concatenation, and each scan's winner
    constexpr int XP = EL + 4, TMAX = 32 * NG;
    constexpr int kWarpFloats = 2 * 32 * XP + TMAX * 4 + TMAX + TMAX * 2;
    float *const wbase = reinterpret_cast<float *>(gridh) + state_words + (threadIdx.x >> 5) * kWarpFloats;
    float *const xs = wbase, *const ws = wbase + 32 * XP;
    ScanTask *const tasks = reinterpret_cast<ScanTask *>(wbase + 2 * 32 * XP);
    unsigned long long *const winner = reinterpret_cast<unsigned long long *>(wbase + 2 * 32 * XP + TMAX * 4);
    uint32_t *const first = reinterpret_cast<uint32_t *>(wbase + 2 * 32 * XP + TMAX * 4 + TMAX * 2);

    const int lane = threadIdx.x & 31, j = lane & (W - 1), gbase = lane & ~(W - 1);
    const int half = lane & (LPB - 1), pbase = lane & ~(LPB - 1), jb = j / LPB;  // lane within its block, block within its super-block
    // a warp takes 32 lanes' worth of elements at a time; the launch gives every warp one such chunk, or, under the
    // CTAs that stay, as many as it takes
    const int64_t nchunks = (nlanes + 31) >> 5;
    for (int64_t chunk = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); chunk < nchunks;
         chunk = (T::LISTS_SHARED || T::LISTS_HOT) ? chunk + (int64_t)gridDim.x * (kThreads / 32) : nchunks) {
    int64_t ln = chunk * 32 + lane;
    const bool active = ln < nlanes;
    if (!active) ln = nlanes - W + j;  // lanes past the end redo the last super-block (whole super-blocks per row) and write nothing
    float xb[EL];
    load_group<EL>(src + ln * EL, xb);

    // sum of squares over the super-block, in element order (lane to lane)
    float sumx2 = 0.f;
#pragma unroll 1
    for (int s = 0; s < W; ++s) {
        if (j == s) {
#pragma unroll
            for (int i = 0; i < EL; ++i) sumx2 += xb[i] * xb[i];
        }
        sumx2 = __shfl_sync(kFull, sumx2, gbase + s);
    }
    const float sigma2 = T::SIGMA_X2 ? 2 * sumx2 / QK_K : sumx2 / QK_K;

    float weight[EL], waux[EL], xval[EL];
    if (qw) {
        const float *qwp = qw + (ln * EL) % n_per_row;
#pragma unroll
        for (int i = 0; i < EL; ++i) weight[i] = __ldg(qwp + i) * sqrtf(sigma2 + xb[i] * xb[i]);
    } else {
#pragma unroll
        for (int i = 0; i < EL; ++i) weight[i] = TYPE == GGML_TYPE_IQ2_S ? 0.25f * sigma2 + xb[i] * xb[i] : xb[i] * xb[i];
    }
#pragma unroll
    for (int i = 0; i < EL; ++i) waux[i] = sqrtf(weight[i]);

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
    // the block's maximum, folded in element order (the first lane of a block starts the fold, the next continues it)
    float max = 0.f;
#pragma unroll
    for (int h = 0; h < LPB; ++h) {
        if (half == h) {
            if (h == 0) max = xval[0];
#pragma unroll
            for (int i = (h == 0 ? 1 : 0); i < EL; ++i) max = max > xval[i] ? max : xval[i];
        }
        if (LPB > 1) max = __shfl_sync(kFull, max, pbase + h);
    }
    {
#pragma unroll
        for (int v = 0; v < EL / 4; ++v) {
            *reinterpret_cast<float4 *>(xs + lane * XP + 4 * v) = make_float4(xval[4 * v], xval[4 * v + 1], xval[4 * v + 2], xval[4 * v + 3]);
            *reinterpret_cast<float4 *>(ws + lane * XP + 4 * v) = make_float4(waux[4 * v], waux[4 * v + 1], waux[4 * v + 2], waux[4 * v + 3]);
        }
        __syncwarp();
    }

    uint32_t L[EL / 4];
#pragma unroll
    for (int i = 0; i < EL / 4; ++i) L[i] = 0;
    float scale = 0.f;
    bool skipped = T::EPS > 0.f ? (max < T::EPS) : !(max != 0.f);
    float eff_max = max;
    if constexpr (T::QP_INIT) {
        if (!skipped) {
            int Linit[EL];
            scale = qp_quants_reg<EL>(T::KMAXQ + 1, xval, Linit, weight);
            eff_max = scale * T::KMAXQ;
            if (eff_max <= 0) {
                skipped = true;
                scale = 0.f;
            } else {
#pragma unroll
                for (int i = 0; i < EL; ++i) lset(L, i, Linit[i]);
            }
        }
    }
    int gidx[NG];
#pragma unroll
    for (int k = 0; k < NG; ++k) gidx[k] = 0;

    {
        // Every lane rounds its groups for one candidate, the warp runs all the scans that came up with the
        // work spread evenly over the lanes, then every block adds up its candidate and accepts or rejects it.
        // the magnitudes are read back from the lane's staged row from here on, which frees their registers
        const float *const xrow = xs + lane * XP;
        // rounds the groups selected by `want` at inverse scale id and looks the lattice points up: a codebook entry
        // (>= 0) or, negative, where the point's neighbour list is and how long
        auto lookup = [&](uint32_t want, float id, int (&g)[NG]) {
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                g[k] = 0;
                if ((want >> k) & 1) {
                    uint32_t u = 0;
                    float xk[GD];
                    load_staged<GD>(xrow + GD * k, xk);
#pragma unroll
                    for (int i = 0; i < GD; ++i) {
                        const int l = imax(0, imin(T::KMAXQ - 1, nearest_int(0.5f * (id * xk[i] - 1))));
                        u |= (uint32_t)l << (T::BITS * i);
                    }
                    g[k] = __ldg(tab.map_s + u);
                }
            }
        };
        // queues the scans of the looked-up groups and runs them; g[] becomes the codebook entry of every group;
        // returns the mask of groups that needed a scan
        auto project = [&](float at_scale, int (&g)[NG]) -> uint32_t {
            uint32_t off = 0, total_n = 0;
            uint32_t nk[NG];
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                nk[k] = 0;
                if (g[k] < 0) {
                    const uint32_t v = (uint32_t)(-g[k] - 1);
                    if ((v & 255u) == 0) {
                        g[k] = 0;  // an empty list (no codebook has one) is not queued
                    } else {
                        off |= 1u << k;
                        nk[k] = v & 255u;
                        g[k] = (int)(v >> 8);  // the list's first record until the winner replaces it
                        total_n += nk[k];
                    }
                }
            }
            // slots and positions: one inclusive scan over (records << 10 | scans)
            const uint32_t mine = (total_n << 10) | (uint32_t)__popc(off);
            uint32_t incl = mine;
#pragma unroll
            for (int dlt = 1; dlt < 32; dlt <<= 1) {
                const uint32_t o = __shfl_up_sync(kFull, incl, dlt);
                if (lane >= dlt) incl += o;
            }
            const uint32_t all = __shfl_sync(kFull, incl, 31);
            uint32_t slot = (incl - mine) & 1023u, pos = (incl - mine) >> 10;
            const uint32_t slot0 = slot;
            __syncwarp();  // the previous round's winners have been read
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                if ((off >> k) & 1) {
                    ScanTask tk;
                    tk.base = (uint32_t)g[k];
                    tk.nrec = nk[k];
                    tk.scale = at_scale;
                    tk.xoff = (uint32_t)(lane * XP + GD * k);
                    tasks[slot] = tk;
                    first[slot] = pos;
                    winner[slot] = kNoWinner;
                    ++slot;
                    pos += nk[k];
                }
            }
            __syncwarp();
            if (all >> 10) balanced_scan<GD, TMAX, T::REC, T::LISTS_SHARED, T::LISTS_HOT>(lane, (int)(all & 1023u), all >> 10, tasks, first, winner, xs, ws, gridh, records,
                                                                                     T::LISTS_HOT ? (uint32_t)tab.hot_bytes / (8 * T::REC) : 0u, T::LISTS_HOT ? tab.records : nullptr);
            __syncwarp();
            slot = slot0;
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                if ((off >> k) & 1) {
                    const uint32_t w = ((uint32_t)winner[slot++] & 0xFFFFu) / (GD * 2);  // row offset -> codebook index
                    g[k] = w < (uint32_t)tab.grid_size ? (int)w : 0;
                }
            }
            return off;
        };
        constexpr uint32_t kAllGroups = NG == 32 ? 0xFFFFFFFFu : ((1u << NG) - 1);
        constexpr int NC = 2 * T::IS_MAX + 1;  // candidate scales; one more pass re-projects at the accepted scale
        auto inverse_scale = [&](int is) { return ((float)(2 * T::KMAXQ - 1) + (float)is * T::STEP) / eff_max; };
        float best = 0;
        if (!T::QP_INIT && !skipped) scale = max / (2 * T::KMAXQ - 1);
        uint32_t on_grid = TYPE == GGML_TYPE_IQ3_S ? 0u : 0xFFFFFFFFu;
        bool reproject = false;
        uint32_t want = 0;
        // the look-ups of candidate is + 1 are issued before the scans of candidate is run
        int g_ahead[NG];
        lookup(skipped ? 0u : kAllGroups, inverse_scale(-T::IS_MAX), g_ahead);
        // pass NC is the re-projection at the accepted scale: all groups (IQ2_XXS, IQ3_S) or those the accepted
        // candidate scanned
        auto one_pass = [&](const int it, const bool last) {
            const float this_scale = last ? scale : 1 / inverse_scale(it - T::IS_MAX);
            int g[NG];
#pragma unroll
            for (int k = 0; k < NG; ++k) g[k] = g_ahead[k];
            if (it + 1 < NC) lookup(skipped ? 0u : kAllGroups, inverse_scale(it + 1 - T::IS_MAX), g_ahead);
            const uint32_t off = project(this_scale, g);
            if (last && reproject) {
#pragma unroll
                for (int k = 0; k < NG; ++k) {
                    if ((want >> k) & 1) {
                        float q[GD];
                        grid_entry<GD>(gridh, g[k], q);
#pragma unroll
                        for (int i = 0; i < GD; ++i) lset(L, GD * k + i, ((int)q[i] - 1) >> 1);
                    }
                }
            }
            // The block's two sums in element order.  The products do not depend on the sums, so every lane forms
            // its own first; with two lanes per block the first lane then adds its terms, hands the sums on, and the
            // second continues (the shuffles are executed by every lane).
            float tx[EL], t2[EL];
            float sumqx = 0, sumq2 = 0;
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                float q[GD], xk[GD];
                if (last) {
#pragma unroll
                    for (int i = 0; i < GD; ++i) q[i] = (float)(2 * lget(L, GD * k + i) + 1);
                } else {
                    grid_entry<GD>(gridh, g[k], q);
                }
                load_staged<GD>(xrow + GD * k, xk);
#pragma unroll
                for (int i = 0; i < GD; ++i) {
                    const float w = weight[GD * k + i];
                    tx[GD * k + i] = w * xk[i] * q[i];
                    t2[GD * k + i] = w * q[i] * q[i];
                    if (LPB == 1) { sumqx += tx[GD * k + i]; sumq2 += t2[GD * k + i]; }
                }
            }
            if (LPB > 1) {
#pragma unroll
                for (int h = 0; h < LPB; ++h) {
                    if (half == h) {
#pragma unroll
                        for (int i = 0; i < EL; ++i) { sumqx += tx[i]; sumq2 += t2[i]; }
                    }
                    sumqx = __shfl_sync(kFull, sumqx, pbase + h);
                    sumq2 = __shfl_sync(kFull, sumq2, pbase + h);
                }
            }
            if (last) {
                if (reproject && sumq2 > 0) scale = sumqx / sumq2;
                return;
            }
            if (!skipped && sumq2 > 0 && sumqx * sumqx > best * sumq2) {
                scale = sumqx / sumq2;
                best = scale * sumqx;
#pragma unroll
                for (int k = 0; k < NG; ++k) {
                    float q[GD];
                    grid_entry<GD>(gridh, g[k], q);
#pragma unroll
                    for (int v = 0; v < GD / 4; ++v)
                        L[(GD * k) / 4 + v] = (uint32_t)(((int)q[4 * v] - 1) >> 1) | ((uint32_t)(((int)q[4 * v + 1] - 1) >> 1) << 8) |
                                              ((uint32_t)(((int)q[4 * v + 2] - 1) >> 1) << 16) | ((uint32_t)(((int)q[4 * v + 3] - 1) >> 1) << 24);
                }
                on_grid = ~off;
            }
            if (it == NC - 1) {
                bool any_off = !skipped && (on_grid & kAllGroups) != kAllGroups;
                if (LPB > 1) any_off = ((__ballot_sync(kFull, any_off) >> pbase) & ((1u << LPB) - 1)) != 0;  // either lane of the block
                if (!skipped) reproject = TYPE == GGML_TYPE_IQ2_XXS ? scale > 0 : (any_off && scale > 0);
                constexpr bool all_groups = TYPE == GGML_TYPE_IQ2_XXS || TYPE == GGML_TYPE_IQ3_S;
                want = reproject ? (all_groups ? kAllGroups : (~on_grid & kAllGroups)) : 0u;
                lookup(want, reproject ? 1 / scale : 0.f, g_ahead);
            }
        };
        if constexpr (T::MERGED) {  // the re-projection runs through the candidates' copy of the scan code
#pragma unroll 1
            for (int it = 0; it <= NC; ++it) one_pass(it, it == NC);
        } else {                    // it gets a copy of its own
#pragma unroll 1
            for (int it = 0; it < NC; ++it) one_pass(it, false);
            one_pass(NC, true);
        }
        if (!skipped) {
            if (scale < 0) {
                scale = -scale;
#pragma unroll
                for (int k = 0; k < NS; ++k) signs[k] = T::PARITY ? (~signs[k]) & 127 : (~signs[k]) & 0xFF;
            }
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                uint32_t u = 0;
#pragma unroll
                for (int i = 0; i < GD; ++i) u |= (uint32_t)lget(L, GD * k + i) << (T::BITS * i);
                const int m = __ldg(tab.map + u);
                gidx[k] = m < 0 ? 0 : m;
            }
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
    const int lsc_next = __shfl_down_sync(kFull, lsc, LPB);  // the next block's
    // position of this block's payload for the format whose writer does not advance over skipped blocks
    const unsigned group_mask = (W == 32) ? kFull : (((1u << W) - 1) << gbase);
    const unsigned live = __ballot_sync(kFull, !skipped && half == 0) & group_mask;  // one bit per block
    const int nlive = __popc(live);
    const int rank_live = __popc(live & ((1u << pbase) - 1));
    const int rank_dead = jb - rank_live;
    // bits a block's first lane needs from its second (IQ3: index and sign bits of the block's upper half), or
    // IQ2_S: two bits per group of eight go to qh[ib/2], gathered from the neighbour lane
    uint32_t hi_bits = 0;
    if (TYPE == GGML_TYPE_IQ2_S) hi_bits = (uint32_t)(gidx[0] >> 8) | ((uint32_t)(gidx[NG > 1 ? 1 : 0] >> 8) << 2);
    if (TYPE == GGML_TYPE_IQ3_XXS) hi_bits = signs[0] | (signs[NS > 1 ? 1 : 0] << 7);
    if (TYPE == GGML_TYPE_IQ3_S) {
#pragma unroll
        for (int k = 0; k < NG; ++k) hi_bits |= (uint32_t)(gidx[k] >> 8) << k;
    }
    const uint32_t hi_next = __shfl_down_sync(kFull, hi_bits, 1);
    if (!active) continue;

    uint8_t *out = dst + (ln / W) * T::BYTES;
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
        static_assert(TYPE != GGML_TYPE_IQ3_XXS || (LPB == 2 && NG == 4 && NS == 2), "two lanes of four groups per block");
#pragma unroll
        for (int k = 0; k < NG; ++k) out[2 + 8 * jb + NG * half + k] = (skipped || clear_all) ? 0 : (uint8_t)gidx[k];
        if (half == 0) {
            uint32_t sas = 0;
            if (!skipped && !clear_all) sas = hi_bits | (hi_next << 14);
            if (!clear_all) sas |= (uint32_t)lsc << 28;
            st32(out + 2 + 64 + 4 * jb, sas);
        }
    } else {  // IQ3_S: payload slots are consumed only by blocks that were not skipped
        static_assert(TYPE != GGML_TYPE_IQ3_S || (LPB == 2 && NG == 4 && NS == 2), "two lanes of four groups per block");
        const int pos = skipped ? nlive + rank_dead : rank_live;
#pragma unroll
        for (int k = 0; k < NG; ++k) out[2 + 8 * pos + NG * half + k] = skipped ? 0 : (uint8_t)gidx[k];
        if (half == 0) out[66 + jb] = skipped ? 0 : (uint8_t)(hi_bits | (hi_next << NG));
#pragma unroll
        for (int k = 0; k < NS; ++k) out[74 + 4 * pos + NS * half + k] = skipped ? 0 : (uint8_t)signs[k];
        if (half == 0 && (jb & 1) == 0) out[106 + (jb >> 1)] = empty ? 0 : (uint8_t)(lsc | (lsc_next << 4));
    }
    }  // chunks
}

template <int TYPE>
cudaError_t launch(const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row, const DeviceState *state,
                   cudaStream_t stream) {
    using T = Traits<TYPE>;
    const IqSearchTable &tab = state->iq[T::TABLE];
    if (!tab.grid || !tab.records || !tab.map_s || tab.record_steps != T::REC || (tab.hot_bytes & 15) ||
        (T::LISTS_SHARED && tab.hot_bytes != tab.records_bytes))
        return cudaErrorInvalidValue;
    constexpr int EL = T::BS / T::LPB;  // elements per lane
    const int64_t nlanes = nelems / EL;
    if (nlanes <= 0) return cudaSuccess;
    constexpr int kThreads = T::THREADS, NG = EL / T::GD, XP = EL + 4, TMAX = 32 * NG;
    int64_t grid = (nlanes + kThreads - 1) / kThreads;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    size_t smem = ((size_t)tab.grid_size * T::GD / 2 + (kThreads / 32) * (2 * 32 * XP + TMAX * 7)) * sizeof(float);
    if (T::LISTS_SHARED || T::LISTS_HOT) {  // one CTA per SM for the whole launch
        static const int sms = [] {
            int dev = 0, n = 148;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            return n > 0 ? n : 1;
        }();
        if (grid > sms) grid = sms;
        smem += (size_t)tab.hot_bytes;
    }
    // a per-device setting: made on every launch (microseconds against a kernel of milliseconds) so that every GPU
    // of a process that drives several has it
    const cudaError_t attr = cudaFuncSetAttribute(quant_iq23_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (attr != cudaSuccess) return attr;
    quant_iq23_kernel<TYPE><<<(unsigned)grid, kThreads, smem, stream>>>(src, qw, static_cast<uint8_t *>(dst), nlanes, n_per_row, tab);
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
