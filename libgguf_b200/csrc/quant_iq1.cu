// Ternary lattice quantizers IQ1_S (32-element blocks) and IQ1_M (16-element blocks).
//
// One thread per block.  The upstream algorithm sorts the block's values (here: by counting ranks
// in registers), then searches all split points (i1 <= i2) of the sorted order into the three
// levels {-1, 0, +1} (+- a fixed shift), keeping the split with the best weighted projection score;
// the accept/reject chain is order dependent through fp32 rounding, so it is replayed sequentially.
// The winning level pattern of each group of eight is then mapped to the 2048-entry codebook,
// through the neighbour lists when it is not a codebook point: those scans are pooled per warp and
// spread evenly over its lanes.  Arrays that are indexed by data (the sorted order, the prefix sums,
// the level scatter) live in shared memory, laid out [index][thread] so that the uniform loops of a
// warp hit one row; everything indexed statically stays in registers; the scans reuse that memory.
// upstream: csrc/quant/iq1_s.cpp:6-204, iq1_m.cpp:4-318, libgguf_iq_tables.cpp:714-789.
#include <float.h>
#include <math.h>

#include "device_state.h"
#include "gguf_common.cuh"
#include "kernels.h"

namespace gguf {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kThreads = 64;

GGUF_D void st16(uint8_t *p, uint32_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

template <int N>
GGUF_D void load_group(const float *p, float (&x)[N]) {
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p) + k);
        x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
    }
}

// The neighbour scans (upstream libgguf_iq_tables.cpp:714-781, the reachable part: a non-empty list) of a warp's 32
// blocks, run the way the IQ2 / IQ3 kernels run theirs: every lane stages its block's values and weights in a padded
// shared-memory row and queues a task per group that is off the codebook; the lists (kept as aligned records of four
// entries whose tails repeat their first entry, an entry being 16 x its codebook index) are laid end to end and every
// lane evaluates an equal stretch of records, whatever lists it crosses.  A list's winner is the first strict minimum
// in list order = the minimum of (distance bits, position) as one 64-bit key (distances are sums of non-negative
// terms, so their bit patterns order like the values; FLT_MAX and NaN never win, as upstream's `<` against FLT_MAX);
// a lane that saw a whole list stores its key, lanes that share one combine theirs with a shared-memory atomic
// minimum.  With one list at a time and all 32 lanes on it (16 shuffles to hand the group over, lists of 1 to 205
// entries, two warp-wide minima per list) the scans were a fifth of the instructions and half of the time.
struct alignas(16) ScanTask {
    uint32_t base;   // the list's first record in the record array
    uint32_t nrec;   // its length in records
    float scale;
    uint32_t xoff;   // float offset of the group in the warp's staged rows; bit 31: the +1/8 levels (else -1/8)
};
constexpr unsigned long long kNoWinner = ~0ull;

GGUF_D uint32_t umin_(uint32_t a, uint32_t b) { return a < b ? a : b; }

template <int TMAX>
GGUF_D void balanced_scan(int lane, int T, uint32_t S, const ScanTask *tasks, const uint32_t *first, unsigned long long *winner,
                          const float *xs, const float *ws, const uint8_t *__restrict__ grid, const uint2 *__restrict__ recs) {
    constexpr int AHEAD = 3;  // records are fetched this many iterations early, across list boundaries
    const uint32_t share = (S + 31) >> 5;
    uint32_t s = umin_((uint32_t)lane * share, S);
    const uint32_t end = umin_(s + share, S);
    if (s >= end) return;
    int t = 0;
#pragma unroll
    for (int step = TMAX / 2; step; step >>= 1) {
        const int c = t + step;
        if (c < T && first[c] <= s) t = c;
    }
    ScanTask tk;
    float2 nx[4], wv[4];
    float sq0, sq1, sq2;   // scale times the three level values
    auto take = [&](int which) {
        tk = tasks[which];
        const float *xr = xs + (tk.xoff & 0x7FFFFFFFu), *wr = ws + (tk.xoff & 0x7FFFFFFFu);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float4 a = reinterpret_cast<const float4 *>(xr)[k], b = reinterpret_cast<const float4 *>(wr)[k];
            nx[2 * k] = make_float2(-a.x, -a.y); nx[2 * k + 1] = make_float2(-a.z, -a.w);
            wv[2 * k] = make_float2(b.x, b.y); wv[2 * k + 1] = make_float2(b.z, b.w);
        }
        const float shift = (tk.xoff >> 31) ? 0.125f : -0.125f;
        sq0 = tk.scale * (-1.f + shift);
        sq1 = tk.scale * shift;
        sq2 = tk.scale * (1.f + shift);
    };
    take(t);
    uint32_t j = s - first[t];
    bool whole = j == 0;
    float best_d2 = FLT_MAX;
    uint32_t best_at = 0xFFFFFFFFu;
    int ft = t;
    uint32_t fleft = tk.nrec - j, fs = s;
    const uint2 *fp = recs + tk.base + j;
    uint2 ring[AHEAD];
    auto fetch = [&](uint2 &rec) {
        if (fs < end) {
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
    for (int d = 0; d < AHEAD; ++d) { ring[d] = make_uint2(0u, 0u); fetch(ring[d]); }
    while (s < end) {
        const uint2 rec = ring[0];
#pragma unroll
        for (int d = 0; d + 1 < AHEAD; ++d) ring[d] = ring[d + 1];
        fetch(ring[AHEAD - 1]);
        const uint32_t at[4] = {rec.x & 0xFFFFu, rec.x >> 16, rec.y & 0xFFFFu, rec.y >> 16};
        float d2[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            // the codebook row: eight bytes 1, 3 or 5 = level 0, 1 or 2 (bit 2 set: level 2, bit 1 set: level 1)
            const uint2 row = __ldg(reinterpret_cast<const uint2 *>(grid + (at[q] >> 1)));
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t w = i < 2 ? row.x : row.y;
                const uint32_t b0 = w >> (16 * (i & 1)), b1 = w >> (16 * (i & 1) + 8);
                const float qa = (b0 & 4u) ? sq2 : ((b0 & 2u) ? sq1 : sq0);
                const float qb = (b1 & 4u) ? sq2 : ((b1 & 2u) ? sq1 : sq0);
                const float2 diff = __fadd2_rn(make_float2(qa, qb), nx[i]);
                const float2 term = __fmul2_rn(__fmul2_rn(wv[i], diff), diff);
                acc = __fadd_rn(acc, term.x);
                acc = __fadd_rn(acc, term.y);
            }
            d2[q] = acc;
        }
        const uint32_t pos = j << 18;  // (entry position of the step) << 16
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (d2[q] < best_d2) { best_d2 = d2[q]; best_at = pos + ((uint32_t)q << 16) + at[q]; }
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
            if (s < end) take(t);
        }
    }
    if (j != 0 && best_d2 < FLT_MAX)
        atomicMin(winner + t, ((unsigned long long)__float_as_uint(best_d2) << 32) | best_at);
}

GGUF_D float level_value(const uint8_t *__restrict__ grid, int index, int i, const float (&xg)[3]) {
    const int c = (__ldg(grid + index * 8 + i) - 1) / 2;
    return c == 0 ? xg[0] : c == 1 ? xg[1] : xg[2];
}

template <int BS>
struct Scratch {
    float ws[BS][kThreads];       // weights, by element
    float pa[BS + 1][kThreads];   // sort keys (the values), then prefix sums of w*x (IQ1_S)
    float pb[BS + 1][kThreads];   // prefix sums of w (IQ1_S)
    uint8_t order[BS][kThreads];  // element index at each sorted position; after the search, the level of each element
};

// Stable ascending insertion sort of the keys in s.pa[0..BS) with their element indices
// (upstream sorts (value, index) pairs with qsort comparing values only; the C library's merge
// sort keeps equal values in index order).
template <int BS>
GGUF_D void sort_block(Scratch<BS> &s, int t) {
    for (int jj = 1; jj < BS; ++jj) {
        const float v = s.pa[jj][t];
        const uint8_t id = s.order[jj][t];
        int p = jj - 1;
        while (p >= 0 && s.pa[p][t] > v) {
            s.pa[p + 1][t] = s.pa[p][t];
            s.order[p + 1][t] = s.order[p][t];
            --p;
        }
        s.pa[p + 1][t] = v;
        s.order[p + 1][t] = id;
    }
}

// The same order by counting: an element's place is the number of elements that sort before it (smaller, or equal with a
// smaller index).  BS x (BS - 1) comparisons on the block's values in registers, no data-dependent loop and no
// shared-memory traffic but the final scatter; the insertion sort above spent about five times the instructions
// shifting keys through shared memory at a different pace in every lane.  Needs comparable values (no NaN).
template <int BS>
GGUF_D void sort_block_by_rank(Scratch<BS> &s, int t, const float (&x)[BS]) {
#pragma unroll
    for (int i = 0; i < BS; ++i) {
        int place = 0;
#pragma unroll
        for (int j = 0; j < BS; ++j) {
            if (j < i) place += x[j] <= x[i] ? 1 : 0;
            if (j > i) place += x[j] < x[i] ? 1 : 0;
        }
        s.pa[place][t] = x[i];
        s.order[place][t] = (uint8_t)i;
    }
}

template <bool IS_M>
__global__ void __launch_bounds__(kThreads, IS_M ? 8 : 7) quant_iq1_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                            uint8_t *__restrict__ dst, int64_t nblocks, int64_t n_per_row,
                                                            IqSearchTable tab) {
    constexpr int BS = IS_M ? 16 : 32, NG = BS / 8, W = 256 / BS, BYTES = IS_M ? 56 : 50;
    __shared__ __align__(16) Scratch<BS> s;
    const int t = threadIdx.x;
    const int lane = t & 31, j = lane & (W - 1), gbase = lane & ~(W - 1);
    int64_t blk = (int64_t)blockIdx.x * kThreads + t;
    const bool active = blk < nblocks;
    if (!active) blk = nblocks - 1;
    float xb[BS], weight[BS];
    load_group<BS>(src + blk * BS, xb);
    const float x_p[3] = {-1 + 0.125f, 0.125f, 1 + 0.125f};
    const float x_m[3] = {-1 - 0.125f, -0.125f, 1 - 0.125f};

    float sumx2 = 0.f;
#pragma unroll 1
    for (int l = 0; l < W; ++l) {
        if (j == l) {
#pragma unroll
            for (int i = 0; i < BS; ++i) sumx2 += xb[i] * xb[i];
        }
        sumx2 = __shfl_sync(kFull, sumx2, gbase + l);
    }
    const float sigma2 = 2 * sumx2 / QK_K;
    if (qw) {
        const float *qwp = qw + (blk * BS) % n_per_row;
#pragma unroll
        for (int i = 0; i < BS; ++i) weight[i] = __ldg(qwp + i) * sqrtf(sigma2 + xb[i] * xb[i]);
    } else {
#pragma unroll
        for (int i = 0; i < BS; ++i) weight[i] = xb[i] * xb[i];
    }
    float max = fabsf(xb[0]);
#pragma unroll
    for (int i = 1; i < BS; ++i) max = max > fabsf(xb[i]) ? max : fabsf(xb[i]);

    float scale = 0.f;
    int shift = IS_M ? 0 : 1;  // IQ1_S: +1 / -1, IQ1_M: sign pattern 0..3
    int index[NG];
#pragma unroll
    for (int k = 0; k < NG; ++k) index[k] = 0;
    bool skipped = max < (IS_M ? 1e-7f : 1e-12f);

    if (!skipped) {
        bool comparable = true;
#pragma unroll
        for (int i = 0; i < BS; ++i) {
            s.ws[i][t] = weight[i];
            comparable = comparable && xb[i] == xb[i];
        }
        if (comparable) {
            sort_block_by_rank<BS>(s, t, xb);
        } else {
#pragma unroll
            for (int i = 0; i < BS; ++i) {
                s.pa[i][t] = xb[i];
                s.order[i][t] = (uint8_t)i;
            }
            sort_block<BS>(s, t);
        }
        float best_score = -FLT_MAX;
        scale = max;
        int besti1 = -1, besti2 = -1, best_k = IS_M ? -1 : 0;
        if constexpr (!IS_M) {
            // prefix sums over the sorted order
            // (the sorted values are the sort keys; each is read before its slot receives a prefix sum)
            float sx = 0.f, sw = 0.f;
            float key = s.pa[0][t];
            s.pa[0][t] = 0.f;
            s.pb[0][t] = 0.f;
            for (int jj = 0; jj < BS; ++jj) {
                const int i = s.order[jj][t];
                const float x = key;
                if (jj + 1 < BS) key = s.pa[jj + 1][t];
                sx = sx + s.ws[i][t] * x;
                sw = sw + s.ws[i][t];
                s.pa[jj + 1][t] = sx;
                s.pb[jj + 1][t] = sw;
            }
            const float sx0 = s.pa[0][t], sw0 = s.pb[0][t], sxn = s.pa[BS][t], swn = s.pb[BS][t];
            for (int i1 = 0; i1 <= BS; ++i1) {
                const float sx1 = s.pa[i1][t], sw1 = s.pb[i1][t];
                for (int i2 = i1; i2 <= BS; ++i2) {
                    const float sx2 = s.pa[i2][t], sw2 = s.pb[i2][t];
                    float sumqx = (sx1 - sx0) * x_p[0] + (sx2 - sx1) * x_p[1] + (sxn - sx2) * x_p[2];
                    float sumq2 = (sw1 - sw0) * x_p[0] * x_p[0] + (sw2 - sw1) * x_p[1] * x_p[1] + (swn - sw2) * x_p[2] * x_p[2];
                    if (sumq2 > 0 && sumqx * sumqx > best_score * sumq2) {
                        scale = sumqx / sumq2; best_score = scale * sumqx; besti1 = i1; besti2 = i2; best_k = 1;
                    }
                    sumqx = (sx1 - sx0) * x_m[0] + (sx2 - sx1) * x_m[1] + (sxn - sx2) * x_m[2];
                    sumq2 = (sw1 - sw0) * x_m[0] * x_m[0] + (sw2 - sw1) * x_m[1] * x_m[1] + (swn - sw2) * x_m[2] * x_m[2];
                    if (sumq2 > 0 && sumqx * sumqx > best_score * sumq2) {
                        scale = sumqx / sumq2; best_score = scale * sumqx; besti1 = i1; besti2 = i2; best_k = -1;
                    }
                }
            }
            if (besti1 < 0 || besti2 < 0 || best_k == 0) skipped = true;
        } else {
            // sorted copies in registers: weight, value, "element is in the first half"
            float wso[BS], xso[BS];
            uint32_t lo_mask = 0;
#pragma unroll
            for (int jj = 0; jj < BS; ++jj) {
                const int i = s.order[jj][t];
                wso[jj] = s.ws[i][t];
                xso[jj] = s.pa[jj][t];
                if (i < BS / 2) lo_mask |= 1u << jj;
            }
            // Upstream adds the 16 terms of each of the eight sums from scratch for every split (i1, i2), in sorted
            // order.  The terms of the positions below i2 do not depend on i2 and those below i1 not on i1 either,
            // so the chains over them are carried from split to split (one more term each time) and only the tail
            // from i2 on (level 2) is added again: the same additions in the same order, 969 term steps instead of 2448.
            struct Sums { float qx0, qx1, qx2, qx3, q20, q21, q22, q23; };
            auto add_term = [&](Sums &S, float w, float x, bool lo, float xp, float xm) {
                const float ap = w * xp * x, am = w * xm * x;
                const float bp = w * xp * xp, bm = w * xm * xm;
                S.qx0 += ap; S.qx1 += lo ? ap : am; S.qx2 += lo ? am : ap; S.qx3 += am;
                S.q20 += bp; S.q21 += lo ? bp : bm; S.q22 += lo ? bm : bp; S.q23 += bm;
            };
#pragma unroll
            for (int jj = 0; jj < BS; ++jj) s.pb[jj][t] = wso[jj];  // sorted weights, for the positions indexed by i1 / i2
            Sums below_i1 = {0, 0, 0, 0, 0, 0, 0, 0};                 // positions < i1 at level 0
            for (int i1 = 0; i1 <= BS; ++i1) {
                Sums below_i2 = below_i1;                             // ... then positions i1 .. i2-1 at level 1
                for (int i2 = i1; i2 <= BS; ++i2) {
                    Sums S = below_i2;
#define GGUF_IQ1M_TAIL(JJ) case JJ: add_term(S, wso[JJ], xso[JJ], (lo_mask >> JJ) & 1, x_p[2], x_m[2]); [[fallthrough]];
                    switch (i2) {
                        GGUF_IQ1M_TAIL(0) GGUF_IQ1M_TAIL(1) GGUF_IQ1M_TAIL(2) GGUF_IQ1M_TAIL(3) GGUF_IQ1M_TAIL(4) GGUF_IQ1M_TAIL(5)
                        GGUF_IQ1M_TAIL(6) GGUF_IQ1M_TAIL(7) GGUF_IQ1M_TAIL(8) GGUF_IQ1M_TAIL(9) GGUF_IQ1M_TAIL(10) GGUF_IQ1M_TAIL(11)
                        GGUF_IQ1M_TAIL(12) GGUF_IQ1M_TAIL(13) GGUF_IQ1M_TAIL(14) GGUF_IQ1M_TAIL(15)
                        default: break;
                    }
#undef GGUF_IQ1M_TAIL
                    const float sqx[4] = {S.qx0, S.qx1, S.qx2, S.qx3}, sq2[4] = {S.q20, S.q21, S.q22, S.q23};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (sq2[k] > 0 && sqx[k] * sqx[k] > best_score * sq2[k]) {
                            scale = sqx[k] / sq2[k]; best_score = scale * sqx[k]; besti1 = i1; besti2 = i2; best_k = k;
                        }
                    }
                    if (i2 < BS) add_term(below_i2, s.pb[i2][t], s.pa[i2][t], (lo_mask >> i2) & 1, x_p[1], x_m[1]);
                }
                if (i1 < BS) add_term(below_i1, s.pb[i1][t], s.pa[i1][t], (lo_mask >> i1) & 1, x_p[0], x_m[0]);
            }
            if (besti1 < 0 || besti2 < 0 || best_k < 0) skipped = true;
        }
        // IQ1_M: the block's values and weights are not kept in registers across the search (the search needs them for
        // itself): the values are read again from the source row, the weights from their scratch rows.  (IQ1_S, whose
        // search works on prefix sums in shared memory, has the registers to keep them.)
        if constexpr (IS_M) {
            load_group<BS>(src + blk * BS, xb);
#pragma unroll
            for (int i = 0; i < BS; ++i) weight[i] = s.ws[i][t];
        }
        if (skipped) {
            scale = 0.f;
        } else {
            // the level of every element: the sorted order is read out, then its column (this thread's own) takes the levels
            uint8_t at_position[BS];
#pragma unroll
            for (int jj = 0; jj < BS; ++jj) at_position[jj] = s.order[jj][t];
#pragma unroll
            for (int jj = 0; jj < BS; ++jj) s.order[at_position[jj]][t] = (uint8_t)(jj < besti1 ? 0 : (jj < besti2 ? 1 : 2));
            int L[BS];
#pragma unroll
            for (int i = 0; i < BS; ++i) L[i] = s.order[i][t];
            if (scale < 0) {
#pragma unroll
                for (int i = 0; i < BS; ++i) L[i] = 2 - L[i];
                scale = -scale;
                best_k = IS_M ? 3 - best_k : -best_k;
            }
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                uint32_t u = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) u |= (uint32_t)L[8 * k + i] << (2 * i);
                index[k] = __ldg(tab.map_s + u);  // negative: off the codebook; where its list is and how long
            }
            shift = best_k;
        }
    }
    // the scans, spread over the warp (balanced_scan above).  The search's scratch arrays are done with: each warp
    // takes half of their memory for its rows, its task queue, the lists' positions and the winners.
    __syncthreads();
    constexpr int XP = BS + 4, TMAX = 32 * NG;
    static_assert(sizeof(Scratch<BS>) / 2 >= (2 * 32 * XP + TMAX * 7) * sizeof(float) && (sizeof(Scratch<BS>) / 2) % 16 == 0, "scratch reuse");
    float *const wbase = reinterpret_cast<float *>(reinterpret_cast<char *>(&s) + (t >> 5) * (sizeof(Scratch<BS>) / 2));
    float *const xs = wbase, *const ws = wbase + 32 * XP;
    ScanTask *const tasks = reinterpret_cast<ScanTask *>(wbase + 2 * 32 * XP);
    unsigned long long *const winner = reinterpret_cast<unsigned long long *>(wbase + 2 * 32 * XP + TMAX * 4);
    uint32_t *const first = reinterpret_cast<uint32_t *>(wbase + 2 * 32 * XP + TMAX * 6);
#pragma unroll
    for (int v = 0; v < BS / 4; ++v) {
        *reinterpret_cast<float4 *>(xs + lane * XP + 4 * v) = make_float4(xb[4 * v], xb[4 * v + 1], xb[4 * v + 2], xb[4 * v + 3]);
        *reinterpret_cast<float4 *>(ws + lane * XP + 4 * v) = make_float4(weight[4 * v], weight[4 * v + 1], weight[4 * v + 2], weight[4 * v + 3]);
    }
    bool all_on_grid = true;
    {
        uint32_t queued = 0, total_n = 0;
        uint32_t nk[NG];
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            nk[k] = 0;
            if (!skipped && index[k] < 0) {
                const uint32_t v = (uint32_t)(-index[k] - 1);
                all_on_grid = false;
                if ((v & 255u) == 0) {
                    index[k] = 0;  // an empty list (the codebook has none) is not queued
                } else {
                    queued |= 1u << k;
                    nk[k] = v & 255u;
                    index[k] = (int)(v >> 8);  // the list's first record until the winner replaces it
                    total_n += nk[k];
                }
            }
        }
        // slots and positions: one inclusive scan over (records << 10 | scans)
        const uint32_t mine = (total_n << 10) | (uint32_t)__popc(queued);
        uint32_t incl = mine;
#pragma unroll
        for (int dlt = 1; dlt < 32; dlt <<= 1) {
            const uint32_t o = __shfl_up_sync(kFull, incl, dlt);
            if (lane >= dlt) incl += o;
        }
        const uint32_t all = __shfl_sync(kFull, incl, 31);
        uint32_t slot = (incl - mine) & 1023u, pos = (incl - mine) >> 10;
        const uint32_t slot0 = slot;
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            if ((queued >> k) & 1) {
                const bool plus = IS_M ? (k == 0 ? shift < 2 : (shift % 2 == 0)) : shift == 1;
                ScanTask tk;
                tk.base = (uint32_t)index[k];
                tk.nrec = nk[k];
                tk.scale = scale;
                tk.xoff = (uint32_t)(lane * XP + 8 * k) | (plus ? 0x80000000u : 0u);
                tasks[slot] = tk;
                first[slot] = pos;
                winner[slot] = kNoWinner;
                ++slot;
                pos += nk[k];
            }
        }
        __syncwarp();
        if (all >> 10)
            balanced_scan<TMAX>(lane, (int)(all & 1023u), all >> 10, tasks, first, winner, xs, ws, tab.grid, static_cast<const uint2 *>(tab.records));
        __syncwarp();
        slot = slot0;
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            if ((queued >> k) & 1) {
                const uint32_t w = ((uint32_t)winner[slot++] & 0xFFFFu) >> 4;  // 16 x index -> index
                index[k] = w < (uint32_t)tab.grid_size ? (int)w : 0;           // nothing comparable: upstream would index with -1
            }
        }
    }
    if (!skipped && !all_on_grid) {
        float sumqx = 0, sumq2 = 0;
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            const bool plus = IS_M ? (k == 0 ? shift < 2 : (shift % 2 == 0)) : shift == 1;
            const float xx[3] = {plus ? x_p[0] : x_m[0], plus ? x_p[1] : x_m[1], plus ? x_p[2] : x_m[2]};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float w = weight[8 * k + i];
                const float q = level_value(tab.grid, index[k], i, xx);
                sumqx += w * q * xb[8 * k + i];
                sumq2 += w * q * q;
            }
        }
        if (sumqx > 0 && sumq2 > 0) scale = sumqx / sumq2;
    }
    if (skipped) { scale = 0.f; shift = IS_M ? 0 : 1; }

    // ---- super-block stage ----
    float max_scale = scale;
#pragma unroll
    for (int m = 1; m < W; m <<= 1) {
        const float o = __shfl_xor_sync(kFull, max_scale, m);
        max_scale = max_scale > o ? max_scale : o;
    }
    const bool empty = !(max_scale != 0.f);
    float d = max_scale / 15;
    const float idd = 1 / d;
    int l = 0;
    if (!empty) l = imax(0, imin(7, nearest_int(0.5f * (idd * scale - 1))));
    uint8_t *out = dst + (blk / W) * BYTES;

    if constexpr (!IS_M) {
        if (!active) return;
        if (j == 0) st16(out, empty ? 0u : f32_to_half_bits(d * 1.125f));
        uint32_t h = 0;
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            out[2 + 4 * j + k] = (uint8_t)index[k];
            h |= (uint32_t)(index[k] >> 8) << (3 * k);
        }
        if (!empty) h |= (uint32_t)(l | (shift == -1 ? 8 : 0)) << 12;
        st16(out + 34 + 2 * j, h);
    } else {
        // refit of the super-block scale over all 256 elements in block order (lane to lane)
        const uint32_t masks[4] = {0x00, 0x80, 0x08, 0x88};
        float sumqx_f = 0.f, sumq2_f = 0.f;
#pragma unroll 1
        for (int sidx = 0; sidx < W; ++sidx) {
            if (j == sidx && !empty) {
#pragma unroll
                for (int k = 0; k < NG; ++k) {
                    const bool plus = k == 0 ? shift < 2 : (shift % 2 == 0);
                    const float xx[3] = {plus ? x_p[0] : x_m[0], plus ? x_p[1] : x_m[1], plus ? x_p[2] : x_m[2]};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float w = weight[8 * k + i];
                        const float q = level_value(tab.grid, index[k], i, xx) * (float)(2 * l + 1);
                        sumqx_f += w * q * xb[8 * k + i];
                        sumq2_f += w * q * q;
                    }
                }
            }
            sumqx_f = __shfl_sync(kFull, sumqx_f, gbase + sidx);
            sumq2_f = __shfl_sync(kFull, sumq2_f, gbase + sidx);
        }
        if (sumq2_f > 0) d = sumqx_f / sumq2_f;
        const uint32_t s16 = empty ? 0u : f32_to_half_bits(d * 1.1125f);
        // scale word w = 3-bit codes of blocks 4w..4w+3 plus one nibble of the fp16 super-scale
        const int l1 = __shfl_down_sync(kFull, l, 1), l2 = __shfl_down_sync(kFull, l, 2), l3 = __shfl_down_sync(kFull, l, 3);
        if (!active) return;
        out[2 * j] = (uint8_t)index[0];
        out[2 * j + 1] = (uint8_t)index[1];
        out[32 + j] = (uint8_t)((index[0] >> 8) | ((index[1] >> 8) << 4) | (empty ? 0u : masks[shift]));
        if ((j & 3) == 0) {
            const int w = j >> 2;
            uint32_t word = 0;
            if (!empty) word = (uint32_t)(l | (l1 << 3) | (l2 << 6) | (l3 << 9)) | (((s16 >> (4 * w)) & 0xF) << 12);
            st16(out + 48 + 2 * w, word);
        }
    }
}

}  // namespace

cudaError_t launch_quantize_iq1(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                                const DeviceState *state, cudaStream_t stream) {
    const IqSearchTable &tab = state->iq[IQT_1S];
    if (!tab.grid || !tab.records || !tab.map_s || tab.record_steps != 1) return cudaErrorInvalidValue;
    const bool is_m = type == GGML_TYPE_IQ1_M;
    const int64_t nblocks = nelems / (is_m ? 16 : 32);
    if (nblocks <= 0) return cudaSuccess;
    const int64_t grid = (nblocks + kThreads - 1) / kThreads;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (is_m) quant_iq1_kernel<true><<<(unsigned)grid, kThreads, 0, stream>>>(src, qw, static_cast<uint8_t *>(dst), nblocks, n_per_row, tab);
    else quant_iq1_kernel<false><<<(unsigned)grid, kThreads, 0, stream>>>(src, qw, static_cast<uint8_t *>(dst), nblocks, n_per_row, tab);
    count_launch();
    return cudaGetLastError();
}

}  // namespace gguf
