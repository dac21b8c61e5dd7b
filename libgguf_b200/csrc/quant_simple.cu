// Memory-bound quantizers: Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q1_0, MXFP4, NVFP4, TQ1_0, TQ2_0
// (the paths taken when no importance weights are given; the weighted legacy variants live
// with the K-quant search code).
//
// 32-element types: every lane loads one float4 (16 B), 8 lanes cover a block, a warp covers
// 4 blocks (512 B of input per warp load).  Block extrema are order-free and are reduced with
// shuffles inside the 8-lane group; the one place where the upstream loop is order sensitive --
// "first element with the largest magnitude" in Q4_0 / Q5_0 -- is reduced on (|v|, index) pairs.
// Each CTA assembles its encoded blocks in shared memory and writes them out as 16-byte vectors.
#include <math.h>

#include "gguf_common.cuh"
#include "gguf_tables.cuh"
#include "kernels.h"
#include "tile_io.cuh"

namespace gguf {
namespace {

constexpr int kThreads = 256;
constexpr unsigned kFull = 0xffffffffu;

// max over the 8 lanes of a block group
GGUF_D float group8_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(kFull, v, 1));
    v = fmaxf(v, __shfl_xor_sync(kFull, v, 2));
    v = fmaxf(v, __shfl_xor_sync(kFull, v, 4));
    return v;
}
GGUF_D float group8_min(float v) {
    v = fminf(v, __shfl_xor_sync(kFull, v, 1));
    v = fminf(v, __shfl_xor_sync(kFull, v, 2));
    v = fminf(v, __shfl_xor_sync(kFull, v, 4));
    return v;
}
GGUF_D uint32_t group8_or(uint32_t v) {
    v |= __shfl_xor_sync(kFull, v, 1);
    v |= __shfl_xor_sync(kFull, v, 2);
    v |= __shfl_xor_sync(kFull, v, 4);
    return v;
}

// Signed value of the first element (lowest index) with the largest magnitude in the 32-element
// block spread over 8 lanes x 4 elements (upstream q4_0.cpp:27-38, q5_0.cpp:29-40).
GGUF_D float group8_first_absmax(const float (&x)[4], int lane8) {
    float amax = 0.0f, vmax = 0.0f;
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = fabsf(x[i]);
        if (amax < a) { amax = a; vmax = x[i]; idx = lane8 * 4 + i; }
    }
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
        const float oa = __shfl_xor_sync(kFull, amax, m);
        const float ov = __shfl_xor_sync(kFull, vmax, m);
        const int oi = __shfl_xor_sync(kFull, idx, m);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; vmax = ov; idx = oi; }
    }
    return vmax;
}

// The 16-way nearest-level scan of the FP4 formats (upstream libgguf_common.h:321-335):
// first index with the smallest |level*e - x|.
GGUF_D int best_index_fp4(float x, float e) {
    int best = 0;
    float best_err = fabsf((float)k_fp4_values[0] * e - x);
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        const float err = fabsf((float)k_fp4_values[i] * e - x);
        if (err < best_err) { best = i; best_err = err; }
    }
    return best;
}

enum class Simple { Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, MXFP4 };

template <Simple K> struct SimpleGeom;
template <> struct SimpleGeom<Simple::Q8_0> { static constexpr int BYTES = 34; };
template <> struct SimpleGeom<Simple::Q4_0> { static constexpr int BYTES = 18; };
template <> struct SimpleGeom<Simple::Q4_1> { static constexpr int BYTES = 20; };
template <> struct SimpleGeom<Simple::Q5_0> { static constexpr int BYTES = 22; };
template <> struct SimpleGeom<Simple::Q5_1> { static constexpr int BYTES = 24; };
template <> struct SimpleGeom<Simple::MXFP4> { static constexpr int BYTES = 17; };

// Nibble pair packing: element j (lanes 0..3 of the group) shares a byte with element j+16
// (lanes 4..7).  Lanes 0..3 write 4 bytes each.
GGUF_D void pack_nibbles(uint8_t *qs, const int (&q)[4], int lane8, bool write) {
    int partner[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) partner[i] = __shfl_xor_sync(kFull, q[i], 4);
    if (write && lane8 < 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qs[lane8 * 4 + i] = (uint8_t)((q[i] & 0xF) | ((partner[i] & 0xF) << 4));
    }
}

GGUF_D uint32_t fifth_bits(const int (&q)[4], int lane8) {
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) bits |= (uint32_t)((q[i] >> 4) & 1) << (lane8 * 4 + i);
    return group8_or(bits);
}

GGUF_D void st16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
GGUF_D void st32(uint8_t *p, uint32_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); p[2] = (uint8_t)(v >> 16); p[3] = (uint8_t)(v >> 24); }

// `mx_steps` : for MXFP4, table of the smallest float in each binade [2^t, 2^(t+1)), t = -149..127,
// for which the host libm's floorf(log2f(x)) already returns t+1 (+inf bits if it never does).
template <Simple K>
__global__ void __launch_bounds__(kThreads) quant32_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                          int64_t nblocks, const float *__restrict__ mx_steps) {
    constexpr int BYTES = SimpleGeom<K>::BYTES;
    constexpr int BLOCKS_PER_ITER = kThreads / 8;  // 32
    constexpr int ITERS = 4;
    constexpr int TILE_BLOCKS = BLOCKS_PER_ITER * ITERS;  // 128 blocks = 4096 elements per CTA
    __shared__ __align__(16) uint8_t stage[TILE_BLOCKS * BYTES + 32];

    const int64_t b0 = (int64_t)blockIdx.x * TILE_BLOCKS;
    const int nb = (int)(nblocks - b0 < TILE_BLOCKS ? nblocks - b0 : TILE_BLOCKS);
    uint8_t *gdst = dst + b0 * BYTES;
    uint8_t *tile = stage + (reinterpret_cast<uintptr_t>(gdst) & 15);
    const int lane8 = threadIdx.x & 7;

    float x[ITERS][4];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int blk = it * BLOCKS_PER_ITER + (threadIdx.x >> 3);
        if (blk < nb) {
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(src + (b0 + blk) * 32) + lane8);
            x[it][0] = v.x; x[it][1] = v.y; x[it][2] = v.z; x[it][3] = v.w;
        } else {
            x[it][0] = x[it][1] = x[it][2] = x[it][3] = 0.0f;
        }
    }

#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int blk = it * BLOCKS_PER_ITER + (threadIdx.x >> 3);
        uint8_t *out = tile + blk * BYTES;
        const float(&v)[4] = x[it];
        int q[4];
        if constexpr (K == Simple::Q8_0) {
            // upstream q8_0.cpp:16-43
            const float amax = group8_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
            const float d = amax / 127.0f;
            const float id = d ? 1.0f / d : 0.0f;
            if (blk < nb) {
                if (lane8 == 0) st16(out, f32_to_half_bits(d));
#pragma unroll
                for (int i = 0; i < 4; ++i) out[2 + lane8 * 4 + i] = (uint8_t)(int8_t)(int)roundf(v[i] * id);
            }
        } else if constexpr (K == Simple::Q4_0) {
            // upstream q4_0.cpp:16-58
            const float vmax = group8_first_absmax(v, lane8);
            const float d = vmax / -8.0f;
            const float id = d ? 1.0f / d : 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = imin(15, cast_f32_to_i8_x86(v[i] * id + 8.5f)) & 0xFF;
            if (blk < nb && lane8 == 0) st16(out, f32_to_half_bits(d));
            pack_nibbles(out + 2, q, lane8, blk < nb);
        } else if constexpr (K == Simple::Q4_1) {
            // upstream q4_1.cpp:16-57
            const float mn = group8_min(fminf(fminf(v[0], v[1]), fminf(v[2], v[3])));
            const float mx = group8_max(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])));
            const float d = (mx - mn) / 15.0f;
            const float id = d ? 1.0f / d : 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = imin(15, cast_f32_to_i8_x86((v[i] - mn) * id + 0.5f)) & 0xFF;
            if (blk < nb && lane8 == 0) { st16(out, f32_to_half_bits(d)); st16(out + 2, f32_to_half_bits(mn)); }
            pack_nibbles(out + 4, q, lane8, blk < nb);
        } else if constexpr (K == Simple::Q5_0) {
            // upstream q5_0.cpp:18-65
            const float vmax = group8_first_absmax(v, lane8);
            const float d = vmax / -16.0f;
            const float id = d ? 1.0f / d : 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = imin(31, cast_f32_to_i8_x86(v[i] * id + 16.5f)) & 0xFF;
            const uint32_t qh = fifth_bits(q, lane8);
            if (blk < nb && lane8 == 0) { st16(out, f32_to_half_bits(d)); st32(out + 2, qh); }
            pack_nibbles(out + 6, q, lane8, blk < nb);
        } else if constexpr (K == Simple::Q5_1) {
            // upstream q5_1.cpp:18-68.  (uint8_t)(float) truncates; the operand is in [0.5, 31.5].
            const float mn = group8_min(fminf(fminf(v[0], v[1]), fminf(v[2], v[3])));
            const float mx = group8_max(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])));
            const float d = (mx - mn) / 31.0f;
            const float id = d ? 1.0f / d : 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = (int)(uint8_t)(int)((v[i] - mn) * id + 0.5f);
            const uint32_t qh = fifth_bits(q, lane8);
            if (blk < nb && lane8 == 0) { st16(out, f32_to_half_bits(d)); st16(out + 2, f32_to_half_bits(mn)); st32(out + 4, qh); }
            pack_nibbles(out + 8, q, lane8, blk < nb);
        } else {  // MXFP4, upstream mxfp4.cpp:17-54
            const float amax = group8_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
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
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = best_index_fp4(v[i], d);
            if (blk < nb && lane8 == 0) out[0] = (uint8_t)e;
            pack_nibbles(out + 1, q, lane8, blk < nb);
        }
    }
    __syncthreads();
    flush_tile(tile, gdst, nb * BYTES, threadIdx.x, kThreads);
}

// NVFP4: 64-element blocks, four 16-element sub-blocks each with a UE4M3 scale
// (upstream nvfp4.cpp:16-55).  4 lanes per sub-block, 16 lanes per block, 2 blocks per warp.
__global__ void __launch_bounds__(kThreads) quant_nvfp4_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                              int64_t nblocks) {
    constexpr int BYTES = 36;
    constexpr int BLOCKS_PER_ITER = kThreads / 16;  // 16
    constexpr int ITERS = 4;
    constexpr int TILE_BLOCKS = BLOCKS_PER_ITER * ITERS;  // 64 blocks = 4096 elements
    __shared__ __align__(16) uint8_t stage[TILE_BLOCKS * BYTES + 32];
    const int64_t b0 = (int64_t)blockIdx.x * TILE_BLOCKS;
    const int nb = (int)(nblocks - b0 < TILE_BLOCKS ? nblocks - b0 : TILE_BLOCKS);
    uint8_t *gdst = dst + b0 * BYTES;
    uint8_t *tile = stage + (reinterpret_cast<uintptr_t>(gdst) & 15);
    const int lane16 = threadIdx.x & 15, sub = lane16 >> 2, lane4 = lane16 & 3;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int blk = it * BLOCKS_PER_ITER + (threadIdx.x >> 4);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (blk < nb) {
            const float4 t = __ldcs(reinterpret_cast<const float4 *>(src + (b0 + blk) * 64) + lane16);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
        const uint8_t ue = f32_to_ue4m3(amax / 6.0f);
        const float d = ue4m3_half_to_f32(ue);
        int q[4], partner[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = best_index_fp4(v[i], d);
        // element j (lanes 0,1 of the sub-block) pairs with element j+8 (lanes 2,3)
#pragma unroll
        for (int i = 0; i < 4; ++i) partner[i] = __shfl_xor_sync(kFull, q[i], 2);
        if (blk < nb) {
            uint8_t *out = tile + blk * BYTES;
            if (lane4 == 0) out[sub] = ue;
            if (lane4 < 2) {
#pragma unroll
                for (int i = 0; i < 4; ++i) out[4 + sub * 8 + lane4 * 4 + i] = (uint8_t)(q[i] | (partner[i] << 4));
            }
        }
    }
    __syncthreads();
    flush_tile(tile, gdst, nb * BYTES, threadIdx.x, kThreads);
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
    const int64_t nblocks = nelems / 32;
    const int64_t grid = (nblocks + 127) / 128;
    if (grid <= 0) return cudaSuccess;
    quant32_kernel<K><<<(unsigned)grid, kThreads, 0, stream>>>(src, static_cast<uint8_t *>(dst), nblocks, mx_steps);
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
        case GGML_TYPE_NVFP4: {
            const int64_t nblocks = nelems / 64;
            if (nblocks <= 0) return cudaSuccess;
            quant_nvfp4_kernel<<<(unsigned)((nblocks + 63) / 64), kThreads, 0, stream>>>(src, out, nblocks);
            count_launch();
            return cudaGetLastError();
        }
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
