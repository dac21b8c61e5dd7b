// Memory-bound quantizers: Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q1_0, MXFP4, NVFP4, TQ1_0, TQ2_0
// (the paths taken when no importance weights are given; the weighted legacy variants live
// with the K-quant search code).
//
// 32-element types: every lane loads one float4 (16 B), 8 lanes cover a block, a warp covers
// 4 blocks (512 B of input per warp load).  Block extrema are order-free and are reduced with
// shuffles inside the 8-lane group; the one place where the upstream loop is order sensitive --
// "first element with the largest magnitude" in Q4_0 / Q5_0 -- is reduced on (|v|, index) pairs.
// Each CTA assembles its encoded blocks in shared memory and writes them out as 16-byte vectors.
#include <float.h>
#include <math.h>

#include "gguf_common.cuh"
#include "gguf_tables.cuh"
#include "kernels.h"
#include "tile_io.cuh"

namespace gguf {
namespace {

constexpr int kThreads = 256;
constexpr unsigned kFull = 0xffffffffu;

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

// Packs the levels of N elements (element j low nibble, element j + N/2 high nibble of byte j).  The
// threshold form is valid for the whole group when it is valid for the group's largest magnitude; the
// scan runs as a rolled loop so that its code exists once per kernel.
template <int N>
GGUF_D void pack_fp4(const float *x, float amax, float e, uint8_t *out) {
    if (fp4_thresholds_valid(amax, e)) {
#pragma unroll
        for (int j = 0; j < N / 2; ++j)
            out[j] = (uint8_t)(best_index_fp4_thresholds(x[j], e) | (best_index_fp4_thresholds(x[j + N / 2], e) << 4));
    } else {
        // x is a register array: select by comparison instead of indexing it dynamically
#pragma unroll 1
        for (int j = 0; j < N / 2; ++j) {
            float lo = 0.f, hi = 0.f;
#pragma unroll
            for (int k = 0; k < N / 2; ++k) {
                if (k == j) { lo = x[k]; hi = x[k + N / 2]; }
            }
            out[j] = (uint8_t)(best_index_fp4_scan(lo, e) | (best_index_fp4_scan(hi, e) << 4));
        }
    }
}

__global__ void selftest_fp4_kernel(float e, unsigned long long *mismatches) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    unsigned long long bad = 0;
    for (uint64_t bits = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; bits < (1ull << 32); bits += stride) {
        const float x = __uint_as_float((uint32_t)bits);
        if (best_index_fp4(x, e) != best_index_fp4_scan(x, e)) ++bad;
    }
    if (bad) atomicAdd(mismatches, bad);
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

// 32-element types (and NVFP4 as two 16-element sub-blocks per thread).  The CTA stages
// 128 x 32 floats in shared memory with coalesced 16-byte loads; then every thread encodes its own
// 32 elements from registers, serially and in upstream's element order (so "first element with
// the largest magnitude" and the like need no cross-lane exchange); the encoded tile is written
// out as 16-byte vectors.
// `mx_steps` : for MXFP4, table of the smallest float in each binade [2^t, 2^(t+1)), t = -149..127,
// for which the host libm's floorf(log2f(x)) already returns t+1 (+inf bits if it never does).
template <Simple K>
__global__ void __launch_bounds__(kBlockThreads) quant32_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                               int64_t nruns, const float *__restrict__ mx_steps) {
    constexpr int BYTES = SimpleGeom<K>::BYTES;
    __shared__ __align__(16) float xin[kBlockThreads * kRowStride];
    __shared__ __align__(16) uint8_t stage[kBlockThreads * BYTES + 32];

    const int64_t r0 = (int64_t)blockIdx.x * kBlockThreads;
    const int nr = (int)(nruns - r0 < kBlockThreads ? nruns - r0 : kBlockThreads);
    uint8_t *gdst = dst + r0 * BYTES;
    uint8_t *tile = stage + (reinterpret_cast<uintptr_t>(gdst) & 15);
    const float4 *g4 = reinterpret_cast<const float4 *>(src + r0 * 32);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int i = k * kBlockThreads + threadIdx.x;  // float4 index inside the tile
        if (i < nr * 8) *reinterpret_cast<float4 *>(xin + (i >> 3) * kRowStride + (i & 7) * 4) = __ldcs(g4 + i);
    }
    __syncthreads();
    if (threadIdx.x < nr) {
        float x[32];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 v = *reinterpret_cast<const float4 *>(xin + threadIdx.x * kRowStride + 4 * k);
            x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
        }
        uint8_t *out = tile + threadIdx.x * BYTES;
        if constexpr (K == Simple::Q8_0) {
            // upstream q8_0.cpp:16-43
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
            const float d = amax / 127.0f;
            const float id = d ? 1.0f / d : 0.0f;
            st16(out, f32_to_half_bits(d));
#pragma unroll
            for (int j = 0; j < 32; ++j) out[2 + j] = (uint8_t)(int8_t)round_half_away(x[j] * id);
        } else if constexpr (K == Simple::Q4_0 || K == Simple::Q5_0) {
            // upstream q4_0.cpp:16-58, q5_0.cpp:18-65
            constexpr bool FIVE = K == Simple::Q5_0;
            float amax = 0.0f, vmax = 0.0f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (amax < fabsf(x[j])) { amax = fabsf(x[j]); vmax = x[j]; }
            }
            const float d = vmax / (FIVE ? -16.0f : -8.0f);
            const float id = d ? 1.0f / d : 0.0f;
            st16(out, f32_to_half_bits(d));
            uint32_t qh = 0;
#pragma unroll
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
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (x[j] < mn) mn = x[j];
                if (x[j] > mx) mx = x[j];
            }
            const float d = (mx - mn) / (FIVE ? 31.0f : 15.0f);
            const float id = d ? 1.0f / d : 0.0f;
            st16(out, f32_to_half_bits(d));
            st16(out + 2, f32_to_half_bits(mn));
            uint32_t qh = 0;
#pragma unroll
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
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
            int e = 0;
            if (amax > 0.0f) {
                // floorf(log2f(amax)) as the host libm computes it: true binade t, plus one when
                // amax has reached the per-binade step recorded by the host.
                const uint32_t bits = f32_to_bits(amax);
                const int bexp = (int)(bits >> 23);  // 255 (inf) converts to 0x80000000 on x86: low byte 0
                const int t = bexp ? bexp - 127 : (31 - __clz((int)(bits & 0x7fffffu))) - 149;
                const int fl = (t >= -149 && t <= 127 && amax >= mx_steps[t + 149]) ? t + 1 : t;
                // (uint8_t)(float): x86 converts through int32 and keeps the low byte.
                e = bexp == 255 ? 0 : (fl - 2 + 127) & 0xFF;
            }
            const float d = e8m0_half_to_f32((uint8_t)e);
            out[0] = (uint8_t)e;
            pack_fp4<32>(x, amax, d, out + 1);
        } else {
            // NVFP4, upstream nvfp4.cpp:16-55: this thread's 32 elements are sub-blocks 2h and 2h+1 of
            // a 64-element block; its 18 staged bytes are 2 scale bytes followed by 16 quant bytes.
#pragma unroll
            for (int sb = 0; sb < 2; ++sb) {
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(x[16 * sb + j]));
                const uint8_t ue = f32_to_ue4m3(amax / 6.0f);
                const float d = ue4m3_half_to_f32(ue);
                out[sb] = ue;
                pack_fp4<16>(x + 16 * sb, amax, d, out + 2 + 8 * sb);
            }
        }
    }
    __syncthreads();
    if constexpr (K == Simple::NVFP4) {
        // un-interleave: block b = runs 2b, 2b+1 -> d[0..1] d[2..3] qs[0..15] qs[16..31]
        __shared__ __align__(16) uint8_t shuffled[kBlockThreads * BYTES + 32];
        uint8_t *tile2 = shuffled + (reinterpret_cast<uintptr_t>(gdst) & 15);
        for (int i = threadIdx.x; i < nr * BYTES; i += kBlockThreads) {
            const int run = i / BYTES, o = i - run * BYTES;
            const int blk = run >> 1, h = run & 1;
            const int pos = o < 2 ? 2 * h + o : 4 + 16 * h + (o - 2);
            tile2[blk * 36 + pos] = tile[i];
        }
        __syncthreads();
        flush_tile(tile2, gdst, nr * BYTES, threadIdx.x, kBlockThreads);
    } else {
        flush_tile(tile, gdst, nr * BYTES, threadIdx.x, kBlockThreads);
    }
}

// Q1_0: 128-element blocks, d = mean |x| with the sum taken in element order, one sign bit per
// element (upstream q1_0.cpp:16-55).  One warp per block: lanes publish |x| to shared memory,
// lane 0 adds them in order, sign bits come from ballots.
__global__ void __launch_bounds__(kThreads) quant_q1_0_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                             int64_t nblocks) {
    __shared__ float absx[kThreads / 32][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t blk = (int64_t)blockIdx.x * (kThreads / 32) + warp;
    if (blk >= nblocks) return;
    const float *x = src + blk * 128;
    uint8_t *out = dst + blk * 18;
    uint32_t sign_words[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float v = x[k * 32 + lane];
        absx[warp][k * 32 + lane] = fabsf(v);
        sign_words[k] = __ballot_sync(kFull, v >= 0.0f);
    }
    __syncwarp();
    if (lane == 0) {
        float sum_abs = 0.0f;
        for (int j = 0; j < 128; ++j) sum_abs += absx[warp][j];
        st16(out, f32_to_half_bits(sum_abs / 128.0f));
    }
    if (lane < 16) out[2 + lane] = (uint8_t)(sign_words[lane >> 2] >> (8 * (lane & 3)));
}

// lroundf(v) for |v| <= 1 results in {-1,0,1}; kept as the library call for exact tie behaviour.
GGUF_D int trit(float v, float id) { return (int)lroundf(v * id) + 1; }

// TQ1_0 / TQ2_0: 256-element blocks, d = max |x| (upstream tq1_0.cpp:16-98, tq2_0.cpp:16-53).
// One warp per block; the block is staged in shared memory because each output byte mixes
// elements 32 (or 16, or 4) apart.
template <bool TQ1>
__global__ void __launch_bounds__(kThreads) quant_ternary_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                                int64_t nblocks) {
    constexpr int BYTES = TQ1 ? 54 : 66;
    __shared__ float xs[kThreads / 32][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t blk = (int64_t)blockIdx.x * (kThreads / 32) + warp;
    if (blk >= nblocks) return;
    const float *x = src + blk * 256;
    uint8_t *out = dst + blk * BYTES;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float v = x[k * 32 + lane];
        xs[warp][k * 32 + lane] = v;
        amax = fmaxf(amax, fabsf(v));
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, m));
    __syncwarp();
    const float d = amax;
    const float id = d ? 1.0f / d : 0.0f;
    const float *xb = xs[warp];
    if constexpr (TQ1) {
        {   // 32 bytes, 5 trits each, elements n*32 + lane
            int q = 0;
#pragma unroll
            for (int n = 0; n < 5; ++n) q = (q * 3 + trit(xb[n * 32 + lane], id)) & 0xFF;
            out[lane] = (uint8_t)((q * 256 + 242) / 243);
        }
        if (lane < 16) {  // 16 bytes, elements 160 + n*16 + lane
            int q = 0;
#pragma unroll
            for (int n = 0; n < 5; ++n) q = (q * 3 + trit(xb[160 + n * 16 + lane], id)) & 0xFF;
            out[32 + lane] = (uint8_t)((q * 256 + 242) / 243);
        }
        if (lane < 4) {  // 4 bytes, 4 trits each, elements 240 + m*4 + lane, then one more *3
            int q = 0;
#pragma unroll
            for (int m = 0; m < 4; ++m) q = (q * 3 + trit(xb[240 + m * 4 + lane], id)) & 0xFF;
            q = (q * 3) & 0xFF;
            out[48 + lane] = (uint8_t)((q * 256 + 242) / 243);
        }
        if (lane == 0) st16(out + 52, f32_to_half_bits(d));
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int q = 0;
#pragma unroll
            for (int n = 0; n < 4; ++n) q += (trit(xb[j * 128 + n * 32 + lane], id) & 3) << (2 * n);
            out[j * 32 + lane] = (uint8_t)q;
        }
        if (lane == 0) st16(out + 64, f32_to_half_bits(d));
    }
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
    const int64_t grid = (nruns + kBlockThreads - 1) / kBlockThreads;
    if (grid <= 0) return cudaSuccess;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    quant32_kernel<K><<<(unsigned)grid, kBlockThreads, 0, stream>>>(src, static_cast<uint8_t *>(dst), nruns, mx_steps);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

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

// Counts the inputs (all 2^32 float bit patterns) for which the threshold form of the FP4 level
// search differs from the 16-way scan at scale e.
cudaError_t selftest_fp4(float e, unsigned long long *device_counter, cudaStream_t stream) {
    selftest_fp4_kernel<<<148 * 8, 256, 0, stream>>>(e, device_counter);
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
        case GGML_TYPE_Q1_0: {
            const int64_t nblocks = nelems / 128;
            if (nblocks <= 0) return cudaSuccess;
            quant_q1_0_kernel<<<(unsigned)((nblocks + 7) / 8), kThreads, 0, stream>>>(src, out, nblocks);
            count_launch();
            return cudaGetLastError();
        }
        case GGML_TYPE_TQ1_0:
        case GGML_TYPE_TQ2_0: {
            const int64_t nblocks = nelems / 256;
            if (nblocks <= 0) return cudaSuccess;
            const unsigned grid = (unsigned)((nblocks + 7) / 8);
            if (type == GGML_TYPE_TQ1_0) quant_ternary_kernel<true><<<grid, kThreads, 0, stream>>>(src, out, nblocks);
            else quant_ternary_kernel<false><<<grid, kThreads, 0, stream>>>(src, out, nblocks);
            count_launch();
            return cudaGetLastError();
        }
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gguf
