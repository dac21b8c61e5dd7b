// fp16 / bf16 source rows -> fp32 on the device, so that a 16-bit checkpoint crosses the host link at
// 2 bytes per element instead of being widened on the CPU first (upstream decodes on the host:
// csrc/quantize_gguf.cpp:1415-1442, decode_bf16_to_f32 / decode_f16_to_f32, then uploads fp32).
// bf16 is a 16-bit shift; fp16 uses the hardware conversion, which like upstream's F16C path is exact
// for every finite value, infinity and quiet NaN.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gguf_common.cuh"
#include "kernels.h"

namespace gguf {
namespace {

constexpr int kThreads = 256;

template <bool BF16>
GGUF_D float widen_one(uint32_t bits16) {
    if (BF16) return __uint_as_float(bits16 << 16);
    return __half2float(__ushort_as_half((unsigned short)bits16));
}

// VEC: 16-byte loads of eight values and two 16-byte stores (both pointers 16-byte aligned); otherwise one
// value per thread and iteration.
template <bool BF16, bool VEC>
__global__ void __launch_bounds__(kThreads) widen_kernel(const uint16_t *__restrict__ src, float *__restrict__ dst, int64_t n) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (VEC) {
        const int64_t nvec = n >> 3;
        const uint4 *s8 = reinterpret_cast<const uint4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        for (int64_t i = tid; i < nvec; i += stride) {
            const uint4 v = __ldcs(s8 + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            float f[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                f[2 * k] = widen_one<BF16>(w[k] & 0xFFFFu);
                f[2 * k + 1] = widen_one<BF16>(w[k] >> 16);
            }
            __stcs(d4 + 2 * i, make_float4(f[0], f[1], f[2], f[3]));
            __stcs(d4 + 2 * i + 1, make_float4(f[4], f[5], f[6], f[7]));
        }
        for (int64_t i = (nvec << 3) + tid; i < n; i += stride) dst[i] = widen_one<BF16>(src[i]);
    } else {
        for (int64_t i = tid; i < n; i += stride) dst[i] = widen_one<BF16>(src[i]);
    }
}

// Importance weights that upstream derives from the data when a type needs them and none are given: for every
// column the sum of squares over the rows, accumulated in row order in fp32 (upstream _libgguf_module.cpp:1210-1220
// accumulate_imatrix_rows; the NumPy expression in upstream __init__.py:186-189 reduces in the same order).  The sum
// of one column is a strictly sequential chain, so the parallelism is the row width; each thread keeps many loads in
// flight.  `acc` is read and written: a matrix can be fed in pieces, first piece onto zeros.
constexpr int kSumsqThreads = 64;
__global__ void __launch_bounds__(kSumsqThreads) sumsq_columns_kernel(const float *__restrict__ rows, int64_t nrows, int64_t n,
                                                                      float *__restrict__ acc) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    const int64_t c = (int64_t)blockIdx.x * kSumsqThreads + threadIdx.x;
    if (c >= n) return;
    float a = acc[c];
    const float *p = rows + c;
    int64_t r = 0;
    constexpr int AHEAD = 32;
    for (; r + AHEAD <= nrows; r += AHEAD) {
        float v[AHEAD];
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) v[k] = __ldcs(p + (r + k) * n);
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) a += v[k] * v[k];
    }
    for (; r < nrows; ++r) {
        const float v = p[r * n];
        a += v * v;
    }
    acc[c] = a;
}

}  // namespace

cudaError_t launch_sumsq_columns(const float *rows, int64_t nrows, int64_t n, float *acc, cudaStream_t stream) {
    if (nrows <= 0 || n <= 0) return cudaSuccess;
    const int64_t grid = (n + kSumsqThreads - 1) / kSumsqThreads;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    const cudaError_t e = launch_overlapped(sumsq_columns_kernel, (unsigned)grid, kSumsqThreads, stream, rows, nrows, n, acc);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

// src_dtype: 1 fp16, 2 bf16 (the codes of LIBGGUF_CUDA_DEQUANTIZE_DTYPE_*).
cudaError_t launch_widen(int src_dtype, const void *src, float *dst, int64_t n, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    if (src_dtype != 1 && src_dtype != 2) return cudaErrorInvalidValue;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    const int64_t work = vec ? (n + 7) / 8 : n;
    int64_t grid = (work + kThreads - 1) / kThreads;
    if (grid > 148 * 16) grid = 148 * 16;
    const uint16_t *s = static_cast<const uint16_t *>(src);
    cudaError_t e;
    if (src_dtype == 2) e = vec ? launch_overlapped(widen_kernel<true, true>, (unsigned)grid, kThreads, stream, s, dst, n)
                                : launch_overlapped(widen_kernel<true, false>, (unsigned)grid, kThreads, stream, s, dst, n);
    else e = vec ? launch_overlapped(widen_kernel<false, true>, (unsigned)grid, kThreads, stream, s, dst, n)
                 : launch_overlapped(widen_kernel<false, false>, (unsigned)grid, kThreads, stream, s, dst, n);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace gguf
