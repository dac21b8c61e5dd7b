// Importance-weighted variants of the legacy 32-element types (Q4_0, Q4_1, Q5_0, Q5_1) and the
// non-linear 4-bit types IQ4_NL / IQ4_XS.  One thread per 32-element block, searches run from
// registers as in search.cuh.
#include <math.h>

#include <mutex>

#include "device_state.h"
#include "gguf_common.cuh"
#include "gguf_tables.cuh"
#include "kernels.h"
#include "search.cuh"

namespace gguf {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kThreads = 128;

GGUF_D void st16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

template <int N>
GGUF_D void load_group(const float *p, float (&x)[N]) {
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p) + k);
        x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
    }
}

// sigma2[row] = (sum of x[j]^2 over the row, added in index order) / n_per_row.
// upstream q4_0.cpp:131-134 (same in q4_1/q5_0/q5_1): the sum is a single left-to-right chain,
// so one warp per row loads 32 values at a time and every lane replays the same 32 additions.
__global__ void __launch_bounds__(kThreads) row_sigma2_kernel(const float *__restrict__ src, float *__restrict__ sigma2,
                                                             int64_t nrows, int64_t n_per_row) {
    const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (row >= nrows) return;
    const int lane = threadIdx.x & 31;
    const float *x = src + row * n_per_row;
    float acc = 0.f;
    for (int64_t base = 0; base < n_per_row; base += 32) {
        const float v = x[base + lane];  // n_per_row is a multiple of 32
        const float sq = v * v;
#pragma unroll
        for (int l = 0; l < 32; ++l) acc += __shfl_sync(kFull, sq, l);
    }
    if (lane == 0) sigma2[row] = acc / (float)n_per_row;
}

// upstream q4_0.cpp:118-150, q4_1.cpp:59-91, q5_0.cpp:67-107, q5_1.cpp:70-112
template <int TYPE>
__global__ void __launch_bounds__(kThreads) legacy_weighted_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                                  const float *__restrict__ sigma2_rows, uint8_t *__restrict__ dst,
                                                                  int64_t nblocks, int64_t n_per_row) {
    const int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (blk >= nblocks) return;
    const int64_t elem = blk * 32;
    const float sigma2 = sigma2_rows[elem / n_per_row];
    const float *qwp = qw + elem % n_per_row;
    float x[32], w[32];
    load_group<32>(src + elem, x);
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = __ldg(qwp + j) * sqrtf(sigma2 + x[j] * x[j]);
    uint32_t L[8];
    constexpr int BYTES = TYPE == GGML_TYPE_Q4_0 ? 18 : TYPE == GGML_TYPE_Q4_1 ? 20 : TYPE == GGML_TYPE_Q5_0 ? 22 : 24;
    uint8_t *out = dst + blk * BYTES;
    uint8_t *qs;
    if constexpr (TYPE == GGML_TYPE_Q4_0 || TYPE == GGML_TYPE_Q5_0) {
        const float d = search_scale_sym<32, true>(x, w, TYPE == GGML_TYPE_Q4_0 ? 8 : 16, L);
        st16(out, f32_to_half_bits(d));
        qs = out + (TYPE == GGML_TYPE_Q4_0 ? 2 : 6);
    } else {
        float the_min;
        const float d = search_scale_min<32, false>(x, w, TYPE == GGML_TYPE_Q4_1 ? 15 : 31, -0.9f, 0.05f, 36, the_min, L);
        st16(out, f32_to_half_bits(d));
        st16(out + 2, f32_to_half_bits(-the_min));
        qs = out + (TYPE == GGML_TYPE_Q4_1 ? 4 : 8);
    }
    uint32_t qh = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int lo = level_at<32>(L, j), hi = level_at<32>(L, j + 16);
        qs[j] = (uint8_t)((lo & 0xF) | ((hi & 0xF) << 4));
        qh |= (uint32_t)((lo >> 4) & 1) << j;
        qh |= (uint32_t)((hi >> 4) & 1) << (j + 16);
    }
    if constexpr (TYPE == GGML_TYPE_Q5_0 || TYPE == GGML_TYPE_Q5_1) {
        uint8_t *p = out + (TYPE == GGML_TYPE_Q5_0 ? 2 : 4);
        p[0] = (uint8_t)qh; p[1] = (uint8_t)(qh >> 8); p[2] = (uint8_t)(qh >> 16); p[3] = (uint8_t)(qh >> 24);
    }
}

// Nearest of the 16 non-linear levels with upstream's rule (libgguf_common.h:301-317): 0 at or below the first
// level, 15 at or above the last (and for NaN), otherwise the bisection's bracket [val[m], val[m+1]) around x,
// the lower level only when it is strictly closer.  The levels are integers, so the bracket of x is the bracket of
// floor(x): `bracket[floor(x) + 127]` replaces the bisection (floor by one round-down add of 2^23 + 127).
// `val`: shared-memory copy of the level table; `bracket`: 240 bytes, entry i = largest m <= 14 with val[m] <= i - 127.
GGUF_D int best_level(const float *val, const uint8_t *bracket, float x) {
    const float xc = fminf(fmaxf(x, -127.f), 112.5f);
    const int m = bracket[__float_as_uint(__fadd_rd(xc, 8388735.f)) & 0xFF];
    int best = (x - val[m] < val[m + 1] - x) ? m : m + 1;
    if (x <= -127.f) best = 0;
    if (!(x < 113.f)) best = 15;
    return best;
}

// IQ4_NL (XS = false, blocks of 32 stand alone) and IQ4_XS (XS = true, 8 blocks per super-block
// with 6-bit block scales).  upstream iq4_nl.cpp:13-152 with ntry = 7 (the path the row API
// takes, iq4_nl.cpp:154-180 and iq4_xs.cpp:190-214).
template <bool XS>
__global__ void __launch_bounds__(kThreads) quant_iq4_kernel(const float *__restrict__ src, const float *__restrict__ qw,
                                                            uint8_t *__restrict__ dst, int64_t nblocks, int64_t n_per_row) {
    __shared__ float val[16];
    __shared__ uint8_t bracket[240];
    if (threadIdx.x < 16) val[threadIdx.x] = (float)k_iq4nl_values[threadIdx.x];
    for (int i = threadIdx.x; i < 240; i += kThreads) {
        int m = 0;
        for (int k = 1; k <= 14; ++k) if ((int)k_iq4nl_values[k] <= i - 127) m = k;
        bracket[i] = (uint8_t)m;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, j8 = lane & 7, gbase = lane & ~7;
    int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = blk < nblocks;
    if (!active) blk = nblocks - 1;
    float x[32], w[32];
    load_group<32>(src + blk * 32, x);

    // sigma2 = (sum of squares over the super-block, in order) * 2/size
    float sigma2 = 0;
    if (XS) {
#pragma unroll 1
        for (int s = 0; s < 8; ++s) {
            if (j8 == s) {
#pragma unroll
                for (int j = 0; j < 32; ++j) sigma2 += x[j] * x[j];
            }
            sigma2 = __shfl_sync(kFull, sigma2, gbase + s);
        }
        sigma2 *= 2.f / 256;
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) sigma2 += x[j] * x[j];
        sigma2 *= 2.f / 32;
    }
    if (qw) {
        const float *qwp = qw + (blk * 32) % n_per_row;
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = __ldg(qwp + j) * sqrtf(sigma2 + x[j] * x[j]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = x[j] * x[j];
    }
    float amax = 0, max = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float ax = fabsf(x[j]);
        if (ax > amax) { amax = ax; max = x[j]; }
    }
    float scale = 0;
    if (!(amax < 1e-15f)) {
        float d = -max / val[0];
        float id = 1 / d;
        float sumqx = 0, sumq2 = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float q = val[best_level(val, bracket, id * x[j])];
            sumqx += w[j] * q * x[j];
            sumq2 += w[j] * q * q;
        }
        d = sumq2 > 0 ? sumqx / sumq2 : 0.f;
        float best = d * sumqx;
        for (int itry = -7; itry <= 7; ++itry) {
            id = ((float)itry + val[0]) / max;
            sumqx = sumq2 = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float q = val[best_level(val, bracket, id * x[j])];
                sumqx += w[j] * q * x[j];
                sumq2 += w[j] * q * q;
            }
            if (sumq2 > 0 && sumqx * sumqx > best * sumq2) {
                d = sumqx / sumq2;
                best = d * sumqx;
            }
        }
        scale = d;
    }

    uint8_t Lb[32];
    if (!XS) {
        uint8_t *out = dst + blk * 18;
        const float id = scale ? 1 / scale : 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) Lb[j] = (uint8_t)best_level(val, bracket, id * x[j]);
        if (!active) return;
        st16(out, f32_to_half_bits(scale));
#pragma unroll
        for (int j = 0; j < 16; ++j) out[2 + j] = (uint8_t)(Lb[j] | (Lb[j + 16] << 4));
    } else {
        // block scale with the largest magnitude, first one on ties
        float a = fabsf(scale), v = scale;
        int idx = j8;
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
            const float oa = __shfl_xor_sync(kFull, a, m);
            const float ov = __shfl_xor_sync(kFull, v, m);
            const int oi = __shfl_xor_sync(kFull, idx, m);
            if (oa > a || (oa == a && oi < idx)) { a = oa; v = ov; idx = oi; }
        }
        const float max_scale = a > 0 ? v : 0.f;  // amax_scale starts at 0 with a strict '>'
        const float d = -max_scale / 32;
        const float id = d ? 1 / d : 0.f;
        int l = nearest_int(id * scale);
        l = imax(-32, imin(31, l));
        const float dl = d * (float)l;
        const float idl = dl ? 1 / dl : 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) Lb[j] = (uint8_t)best_level(val, bracket, idl * x[j]);
        l += 32;
        // gather the 8 scale codes of the super-block
        int codes[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) codes[s] = __shfl_sync(kFull, l, gbase + s);
        if (!active) return;
        uint8_t *out = dst + (blk >> 3) * 136;
        if (j8 == 0) {
            st16(out, f32_to_half_bits(d));
            uint32_t sh = 0;
#pragma unroll
            for (int s = 0; s < 8; ++s) sh |= (uint32_t)(codes[s] >> 4) << (2 * s);
            st16(out + 2, (uint16_t)sh);
#pragma unroll
            for (int s = 0; s < 4; ++s) out[4 + s] = (uint8_t)((codes[2 * s] & 0xF) | ((codes[2 * s + 1] & 0xF) << 4));
        }
        uint8_t *qs = out + 8 + 16 * j8;
#pragma unroll
        for (int j = 0; j < 16; ++j) qs[j] = (uint8_t)(Lb[j] | (Lb[j + 16] << 4));
    }
}

}  // namespace

cudaError_t launch_quantize_legacy_weighted(int type, const float *src, const float *qw, void *dst, int64_t nrows,
                                            int64_t n_per_row, cudaStream_t stream) {
    if (nrows <= 0) return cudaSuccess;
    float *sigma2 = nullptr;
    cudaError_t err = cudaMallocAsync((void **)&sigma2, (size_t)nrows * sizeof(float), stream);
    if (err != cudaSuccess) return err;
    row_sigma2_kernel<<<(unsigned)((nrows + 3) / 4), kThreads, 0, stream>>>(src, sigma2, nrows, n_per_row);
    count_launch();
    const int64_t nblocks = nrows * n_per_row / 32;
    const unsigned grid = (unsigned)((nblocks + kThreads - 1) / kThreads);
    uint8_t *out = static_cast<uint8_t *>(dst);
    switch (type) {
        case GGML_TYPE_Q4_0: legacy_weighted_kernel<GGML_TYPE_Q4_0><<<grid, kThreads, 0, stream>>>(src, qw, sigma2, out, nblocks, n_per_row); break;
        case GGML_TYPE_Q4_1: legacy_weighted_kernel<GGML_TYPE_Q4_1><<<grid, kThreads, 0, stream>>>(src, qw, sigma2, out, nblocks, n_per_row); break;
        case GGML_TYPE_Q5_0: legacy_weighted_kernel<GGML_TYPE_Q5_0><<<grid, kThreads, 0, stream>>>(src, qw, sigma2, out, nblocks, n_per_row); break;
        case GGML_TYPE_Q5_1: legacy_weighted_kernel<GGML_TYPE_Q5_1><<<grid, kThreads, 0, stream>>>(src, qw, sigma2, out, nblocks, n_per_row); break;
        default: cudaFreeAsync(sigma2, stream); return cudaErrorInvalidValue;
    }
    count_launch();
    err = cudaGetLastError();
    const cudaError_t free_err = cudaFreeAsync(sigma2, stream);
    return err != cudaSuccess ? err : free_err;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the importance-weighted legacy quantizer.
//
// The two-kernel scheme above needs one float of scratch per row (the row's mean square).  Here
// that scratch is a fixed array in the library's device image instead of a stream-ordered
// allocation, for callers that must not allocate: code running where the CUDA allocator is off
// limits (inside a memory-pool owner that forbids foreign allocations, under a hard memory
// budget, or in a real-time loop where an allocation's latency is not acceptable).
// Every GPU that loads the library carries the array (kStaticScratchRows * 4 bytes = 256 KiB)
// until the process exits.  All calls share it and it keeps the previous call's contents; each
// call overwrites the entries it uses before reading them, so nothing has to be cleared, but two
// calls whose kernels overlap on the GPU (different streams, or different host threads) race.
constexpr int64_t kStaticScratchRows = 65536;
static __device__ __align__(256) float g_row_scratch[kStaticScratchRows];

// Device address of g_row_scratch on each device.  In host code the array's name is only a
// stand-in; the address a kernel may use comes from cudaGetSymbolAddress, asked once per device
// with that device current.
static float *g_row_scratch_addr[kMaxDevices];
static std::mutex g_row_scratch_lock;

int64_t static_scratch_max_rows() { return kStaticScratchRows; }

cudaError_t launch_quantize_legacy_weighted_static(int type, const float *src, const float *qw, void *dst, int64_t nrows,
                                                   int64_t n_per_row, cudaStream_t stream) {
    if (nrows <= 0) return cudaSuccess;
    if (nrows > kStaticScratchRows) return cudaErrorInvalidValue;
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    float *scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_row_scratch_lock);
        if (!g_row_scratch_addr[dev]) {
            void *p = nullptr;
            err = cudaGetSymbolAddress(&p, g_row_scratch);
            if (err != cudaSuccess) return err;
            g_row_scratch_addr[dev] = static_cast<float *>(p);
        }
        scratch = g_row_scratch_addr[dev];
    }
    row_sigma2_kernel<<<(unsigned)((nrows + 3) / 4), kThreads, 0, stream>>>(src, scratch, nrows, n_per_row);
    count_launch();
    const int64_t nblocks = nrows * n_per_row / 32;
    const unsigned grid = (unsigned)((nblocks + kThreads - 1) / kThreads);
    uint8_t *out = static_cast<uint8_t *>(dst);
    switch (type) {
        case GGML_TYPE_Q4_0: legacy_weighted_kernel<GGML_TYPE_Q4_0><<<grid, kThreads, 0, stream>>>(src, qw, scratch, out, nblocks, n_per_row); break;
        case GGML_TYPE_Q4_1: legacy_weighted_kernel<GGML_TYPE_Q4_1><<<grid, kThreads, 0, stream>>>(src, qw, scratch, out, nblocks, n_per_row); break;
        case GGML_TYPE_Q5_0: legacy_weighted_kernel<GGML_TYPE_Q5_0><<<grid, kThreads, 0, stream>>>(src, qw, scratch, out, nblocks, n_per_row); break;
        case GGML_TYPE_Q5_1: legacy_weighted_kernel<GGML_TYPE_Q5_1><<<grid, kThreads, 0, stream>>>(src, qw, scratch, out, nblocks, n_per_row); break;
        default: return cudaErrorInvalidValue;
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_quantize_iq4(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                                cudaStream_t stream) {
    const int64_t nblocks = nelems / 32;
    if (nblocks <= 0) return cudaSuccess;
    const unsigned grid = (unsigned)((nblocks + kThreads - 1) / kThreads);
    if (type == GGML_TYPE_IQ4_NL) quant_iq4_kernel<false><<<grid, kThreads, 0, stream>>>(src, qw, static_cast<uint8_t *>(dst), nblocks, n_per_row);
    else quant_iq4_kernel<true><<<grid, kThreads, 0, stream>>>(src, qw, static_cast<uint8_t *>(dst), nblocks, n_per_row);
    count_launch();
    return cudaGetLastError();
}

}  // namespace gguf
