// C-ABI layer: the host-pointer functions of include/libgguf.h, the device-pointer functions of
// include/libgguf_cuda_native.h, type tables, per-device state (staging buffers, search tables)
// and the per-type dispatch into the kernel translation units.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <limits>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/libgguf.h"
#include "../../include/libgguf_cuda_native.h"
#include "device_state.h"
#include "gguf_common.cuh"
#include "host_stage.h"
#include "kernels.h"

namespace gguf {

static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

cudaError_t launch_quantize_simple(int type, const float *src, void *dst, int64_t nelems, const float *mx_steps,
                                   cudaStream_t stream);
cudaError_t launch_quantize_k(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                              cudaStream_t stream);
cudaError_t launch_quantize_legacy_weighted(int type, const float *src, const float *qw, void *dst, int64_t nrows,
                                            int64_t n_per_row, cudaStream_t stream);
cudaError_t launch_quantize_iq4(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                                cudaStream_t stream);
cudaError_t launch_quantize_iq(int type, const float *src, const float *qw, void *dst, int64_t nelems, int64_t n_per_row,
                               const DeviceState *state, cudaStream_t stream);

bool quantize_supported(int type) {
    switch (type) {
        case GGML_TYPE_Q4_0: case GGML_TYPE_Q4_1: case GGML_TYPE_Q5_0: case GGML_TYPE_Q5_1: case GGML_TYPE_Q8_0:
        case GGML_TYPE_Q1_0: case GGML_TYPE_MXFP4: case GGML_TYPE_NVFP4: case GGML_TYPE_TQ1_0: case GGML_TYPE_TQ2_0:
        case GGML_TYPE_Q2_K: case GGML_TYPE_Q3_K: case GGML_TYPE_Q4_K: case GGML_TYPE_Q5_K: case GGML_TYPE_Q6_K:
        case GGML_TYPE_IQ4_NL: case GGML_TYPE_IQ4_XS:
        case GGML_TYPE_IQ2_XXS: case GGML_TYPE_IQ2_XS: case GGML_TYPE_IQ2_S: case GGML_TYPE_IQ3_XXS:
        case GGML_TYPE_IQ3_S: case GGML_TYPE_IQ1_S: case GGML_TYPE_IQ1_M:
            return true;
        default:
            return false;
    }
}

static bool needs_imatrix(int type) {
    return type == GGML_TYPE_IQ2_XXS || type == GGML_TYPE_IQ2_XS || type == GGML_TYPE_IQ1_S;
}

// Per-type routing.  `imatrix` (device, n_per_row floats) may be null.
cudaError_t launch_quantize(int type, const float *src, const float *imatrix, void *dst, int64_t nrows,
                            int64_t n_per_row, const DeviceState *state, cudaStream_t stream) {
    const int64_t nelems = nrows * n_per_row;
    switch (type) {
        case GGML_TYPE_Q8_0: case GGML_TYPE_Q1_0: case GGML_TYPE_MXFP4: case GGML_TYPE_NVFP4:
        case GGML_TYPE_TQ1_0: case GGML_TYPE_TQ2_0:
            // upstream ignores importance weights for these (e.g. mxfp4.cpp:108, q8_0.cpp quantize_q8_0)
            return launch_quantize_simple(type, src, dst, nelems, state ? state->mx_steps : nullptr, stream);
        case GGML_TYPE_Q4_0: case GGML_TYPE_Q4_1: case GGML_TYPE_Q5_0: case GGML_TYPE_Q5_1:
            if (imatrix) return launch_quantize_legacy_weighted(type, src, imatrix, dst, nrows, n_per_row, stream);
            return launch_quantize_simple(type, src, dst, nelems, nullptr, stream);
        case GGML_TYPE_Q2_K: case GGML_TYPE_Q3_K: case GGML_TYPE_Q4_K: case GGML_TYPE_Q5_K: case GGML_TYPE_Q6_K:
            return launch_quantize_k(type, src, imatrix, dst, nelems, n_per_row, stream);
        case GGML_TYPE_IQ4_NL: case GGML_TYPE_IQ4_XS:
            return launch_quantize_iq4(type, src, imatrix, dst, nelems, n_per_row, stream);
        case GGML_TYPE_IQ2_XXS: case GGML_TYPE_IQ2_XS: case GGML_TYPE_IQ2_S: case GGML_TYPE_IQ3_XXS:
        case GGML_TYPE_IQ3_S: case GGML_TYPE_IQ1_S: case GGML_TYPE_IQ1_M:
            return launch_quantize_iq(type, src, imatrix, dst, nelems, n_per_row, state, stream);
        default:
            return cudaErrorInvalidValue;
    }
}

static thread_local std::string t_last_error;

}  // namespace gguf

using namespace gguf;

// =================================================================================================
// type tables
extern "C" size_t libgguf_type_size(enum ggml_type type) {
    const BlockGeom g = block_geom((int)type);
    if (g.bytes) return (size_t)g.bytes;
    switch (type) {
        case GGML_TYPE_Q8_1: return 36;   // fp16 d, fp16 s, 32 x int8
        case GGML_TYPE_Q8_K: return 292;  // fp32 d, 256 x int8, 16 x int16
        case GGML_TYPE_F16: case GGML_TYPE_BF16: case GGML_TYPE_I16: return 2;
        case GGML_TYPE_F32: case GGML_TYPE_I32: return 4;
        case GGML_TYPE_F64: case GGML_TYPE_I64: return 8;
        case GGML_TYPE_I8: return 1;
        default: return 0;
    }
}

extern "C" size_t libgguf_row_size(enum ggml_type type, int64_t n_per_row) {
    if (n_per_row <= 0) return 0;
    switch (type) {
        case GGML_TYPE_F32: return (size_t)n_per_row * 4;
        case GGML_TYPE_F16: case GGML_TYPE_BF16: return (size_t)n_per_row * 2;
        default: break;
    }
    const BlockGeom g = block_geom((int)type);
    if (g.elems == 0 || n_per_row % g.elems != 0) return 0;
    return (size_t)(n_per_row / g.elems) * (size_t)g.bytes;
}

extern "C" const char *libgguf_type_name(enum ggml_type type) {
    switch (type) {
        case GGML_TYPE_F32: return "f32";
        case GGML_TYPE_F16: return "f16";
        case GGML_TYPE_Q4_0: return "q4_0";
        case GGML_TYPE_Q4_1: return "q4_1";
        case GGML_TYPE_Q5_0: return "q5_0";
        case GGML_TYPE_Q5_1: return "q5_1";
        case GGML_TYPE_Q8_0: return "q8_0";
        case GGML_TYPE_Q8_1: return "q8_1";
        case GGML_TYPE_Q2_K: return "q2_K";
        case GGML_TYPE_Q3_K: return "q3_K";
        case GGML_TYPE_Q4_K: return "q4_K";
        case GGML_TYPE_Q5_K: return "q5_K";
        case GGML_TYPE_Q6_K: return "q6_K";
        case GGML_TYPE_Q8_K: return "q8_K";
        case GGML_TYPE_IQ2_XXS: return "iq2_xxs";
        case GGML_TYPE_IQ2_XS: return "iq2_xs";
        case GGML_TYPE_IQ3_XXS: return "iq3_xxs";
        case GGML_TYPE_IQ1_S: return "iq1_s";
        case GGML_TYPE_IQ4_NL: return "iq4_nl";
        case GGML_TYPE_IQ3_S: return "iq3_s";
        case GGML_TYPE_IQ2_S: return "iq2_s";
        case GGML_TYPE_IQ4_XS: return "iq4_xs";
        case GGML_TYPE_I8: return "i8";
        case GGML_TYPE_I16: return "i16";
        case GGML_TYPE_I32: return "i32";
        case GGML_TYPE_I64: return "i64";
        case GGML_TYPE_F64: return "f64";
        case GGML_TYPE_IQ1_M: return "iq1_m";
        case GGML_TYPE_BF16: return "bf16";
        case GGML_TYPE_TQ1_0: return "tq1_0";
        case GGML_TYPE_TQ2_0: return "tq2_0";
        case GGML_TYPE_MXFP4: return "mxfp4";
        case GGML_TYPE_NVFP4: return "nvfp4";
        case GGML_TYPE_Q1_0: return "q1_0";
        default: return "unknown";
    }
}

extern "C" bool libgguf_quantize_requires_imatrix(enum ggml_type type) { return needs_imatrix((int)type); }

// =================================================================================================
// host-pointer chunk functions
namespace {

// ---- checked mode (LIBGGUF_B200_CHECKED=1) ------------------------------------------------------------------
// The stand-in for a memory checker on hosts where none can be run: the host-pointer calls put guard bands of
// kGuard bytes directly before and after the bytes a kernel may touch.  The bands around an output are filled with
// a pattern before the launch and compared after it (a write outside the payload changes them); the band after an
// input is filled with 0xFF (NaN patterns), so a read past the end changes the result and shows up in a byte
// comparison with the CPU reference.  A violation is counted in a status word the host reads
// (libgguf_cuda_checked_violations); nothing traps.  Large calls stay on the single-buffer path in this mode.
constexpr size_t kGuard = 4096;
constexpr unsigned char kGuardByte = 0xC5;
std::atomic<uint64_t> g_guard_violations{0};

bool checked_mode() {
    static const bool on = [] {
        const char *env = getenv("LIBGGUF_B200_CHECKED");
        return env && env[0] && env[0] != '0';
    }();
    return on;
}

__global__ void guard_count_kernel(const unsigned char *front, const unsigned char *back, unsigned long long *bad) {
    unsigned n = 0;
    for (unsigned i = threadIdx.x; i < kGuard; i += blockDim.x) n += (front[i] != kGuardByte) + (back[i] != kGuardByte);
    if (n) atomicAdd(bad, (unsigned long long)n);
}

// Grow-only staging buffers of one device for the host-pointer calls.
struct HostCallStaging {
    std::mutex lock;
    void *d_in = nullptr;
    size_t in_cap = 0;
    void *d_out = nullptr;
    size_t out_cap = 0;
    float *d_imatrix = nullptr;
    size_t im_cap = 0;
    cudaStream_t stream = nullptr;
    StageRing ring;  // large calls: pinned slots, host copies overlapped with the device
    unsigned long long *d_bad = nullptr;  // checked mode: guard bytes found changed

    // checked mode: read and clear the device counter after the stream has been synchronised
    void collect_violations() {
        if (!d_bad) return;
        unsigned long long bad = 0;
        if (cudaMemcpy(&bad, d_bad, sizeof(bad), cudaMemcpyDeviceToHost) == cudaSuccess && bad) {
            g_guard_violations.fetch_add(bad);
            cudaMemset(d_bad, 0, sizeof(bad));
        }
    }
    bool ensure_counter() {
        if (!checked_mode() || d_bad) return true;
        if (cudaMalloc((void **)&d_bad, sizeof(*d_bad)) != cudaSuccess) { cudaGetLastError(); return false; }
        return cudaMemset(d_bad, 0, sizeof(*d_bad)) == cudaSuccess;
    }
};
HostCallStaging g_staging[kMaxDevices];

bool grow(void **p, size_t *cap, size_t need) {
    if (checked_mode()) need += 2 * kGuard;   // callers use guarded() to find the payload inside
    if (need <= *cap) return true;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    if (cudaMalloc(p, need) != cudaSuccess) { cudaGetLastError(); return false; }
    *cap = need;
    return true;
}
// payload address inside a buffer obtained with grow()
char *guarded(void *base) { return (char *)base + (checked_mode() ? kGuard : 0); }
// before a launch: pattern around the output payload, NaN bytes after the input payload
cudaError_t guards_arm(char *d_in, size_t in_bytes, char *d_out, size_t out_bytes, cudaStream_t stream) {
    if (!checked_mode()) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(d_out - kGuard, kGuardByte, kGuard, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_out + out_bytes, kGuardByte, kGuard, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_in + in_bytes, 0xFF, kGuard, stream);
    return e;
}
// after the launch (same stream): count changed guard bytes; the caller synchronises the stream afterwards
cudaError_t guards_check(char *d_out, size_t out_bytes, unsigned long long *d_bad, cudaStream_t stream) {
    if (!checked_mode()) return cudaSuccess;
    guard_count_kernel<<<1, 256, 0, stream>>>((const unsigned char *)d_out - kGuard, (const unsigned char *)d_out + out_bytes, d_bad);
    return cudaGetLastError();
}

// Device used by the host-pointer calls: LIBGGUF_CUDA_DEVICE, else the current device.
bool pick_device(int *dev) {
    const char *env = getenv("LIBGGUF_CUDA_DEVICE");
    if (env && env[0]) {
        *dev = atoi(env);
        return cudaSetDevice(*dev) == cudaSuccess;
    }
    return cudaGetDevice(dev) == cudaSuccess;
}

// Rows per staged piece: bounded so that a huge host matrix never needs a huge device buffer.
constexpr size_t kStageBytes = size_t(256) << 20;
// Calls that move at least kPipelineBytes go through the pinned ring in pieces of kPieceBytes.
constexpr size_t kPipelineBytes = size_t(8) << 20;
constexpr size_t kPieceBytes = size_t(16) << 20;

// LIBGGUF_CUDA_HOST_PIPELINE=0 keeps every call on the single-buffer path.
bool pipeline_enabled() {
    static const bool enabled = [] {
        const char *env = getenv("LIBGGUF_CUDA_HOST_PIPELINE");
        return !(env && env[0] == '0') && !checked_mode();
    }();
    return enabled;
}

int64_t piece_rows(size_t in_row, size_t out_row, int64_t nrows) {
    const size_t widest = in_row > out_row ? in_row : out_row;
    int64_t rows = (int64_t)(kPieceBytes / widest);
    if (rows < 1) rows = 1;
    return rows < nrows ? rows : nrows;
}

}  // namespace

extern "C" size_t libgguf_quantize_chunk(enum ggml_type type, const float *src, void *dst, int64_t start, int64_t nrows,
                                         int64_t n_per_row, const float *imatrix) {
    if (nrows <= 0 || !src || !dst) return 0;
    const size_t row_size = libgguf_row_size(type, n_per_row);
    if (row_size == 0 || start < 0 || start % n_per_row != 0) return 0;
    if (needs_imatrix((int)type) && !imatrix) return 0;
    int dev = 0;
    if (!pick_device(&dev) || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return 0; }
    const size_t start_row = (size_t)(start / n_per_row);
    const float *in = src + start;
    char *out = (char *)dst + start_row * row_size;
    HostCallStaging &st = g_staging[dev];
    std::lock_guard<std::mutex> guard(st.lock);
    if (!st.stream && cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); return 0; }

    // plain storage types (upstream libgguf.cpp:347-352 / libgguf_storage.cpp:105-125)
    const bool storage = type == GGML_TYPE_F32 || type == GGML_TYPE_F16 || type == GGML_TYPE_BF16;
    const DeviceState *state = nullptr;
    if (!storage) {
        if (!quantize_supported((int)type)) return 0;
        state = device_state_for((int)type, dev);
        if (!state) return 0;
    }
    // bulk-staged quantizers: a CTA that gave up on a staged copy left rows unwritten; the counter tells
    const bool watch_staging = uses_bulk_staging((int)type);
    unsigned long long timeouts_before = 0;
    if (watch_staging && read_staging_timeouts(&timeouts_before) != cudaSuccess) { cudaGetLastError(); return 0; }
    auto staging_ok = [&]() {
        if (!watch_staging) return true;
        unsigned long long now = 0;
        if (read_staging_timeouts(&now) != cudaSuccess) { cudaGetLastError(); return false; }
        return now == timeouts_before;
    };
    const size_t in_row = (size_t)n_per_row * 4;
    const float *d_im = nullptr;
    if (imatrix && !storage) {
        if (!grow((void **)&st.d_imatrix, &st.im_cap, in_row)) return 0;
        if (cudaMemcpyAsync(st.d_imatrix, imatrix, in_row, cudaMemcpyHostToDevice, st.stream) != cudaSuccess) { cudaGetLastError(); return 0; }
        d_im = st.d_imatrix;
    }
    if ((size_t)nrows * in_row >= kPipelineBytes && pipeline_enabled()) {
        if (d_im && cudaStreamSynchronize(st.stream) != cudaSuccess) { cudaGetLastError(); return 0; }
        const int64_t rpp = piece_rows(in_row, row_size, nrows);
        if (!st.ring.reserve((size_t)rpp * in_row, (size_t)rpp * row_size)) { cudaGetLastError(); return 0; }
        const cudaError_t err = run_staged(st.ring, (const char *)in, in_row, out, row_size, nrows, rpp,
            [&](const void *d_in, void *d_out, int64_t, int64_t nr, cudaStream_t stream) {
                if (storage) return launch_store(type, (const float *)d_in, d_out, nr * n_per_row, stream);
                return launch_quantize((int)type, (const float *)d_in, d_im, d_out, nr, n_per_row, state, stream);
            });
        if (err != cudaSuccess) { cudaGetLastError(); return 0; }
        return staging_ok() ? (size_t)nrows * row_size : 0;
    }
    int64_t rows_per_piece = (int64_t)(kStageBytes / in_row);
    if (rows_per_piece < 1) rows_per_piece = 1;
    if (rows_per_piece > nrows) rows_per_piece = nrows;
    if (!grow(&st.d_in, &st.in_cap, (size_t)rows_per_piece * in_row)) return 0;
    if (!grow(&st.d_out, &st.out_cap, (size_t)rows_per_piece * row_size)) return 0;
    if (!st.ensure_counter()) return 0;
    char *d_in = guarded(st.d_in), *d_out = guarded(st.d_out);
    for (int64_t r0 = 0; r0 < nrows; r0 += rows_per_piece) {
        const int64_t nr = nrows - r0 < rows_per_piece ? nrows - r0 : rows_per_piece;
        cudaError_t err = guards_arm(d_in, (size_t)nr * in_row, d_out, (size_t)nr * row_size, st.stream);
        if (err == cudaSuccess) err = cudaMemcpyAsync(d_in, in + r0 * n_per_row, (size_t)nr * in_row, cudaMemcpyHostToDevice, st.stream);
        if (err == cudaSuccess) {
            if (storage) err = launch_store(type, (const float *)d_in, d_out, nr * n_per_row, st.stream);
            else err = launch_quantize((int)type, (const float *)d_in, d_im, d_out, nr, n_per_row, state, st.stream);
        }
        if (err == cudaSuccess) err = guards_check(d_out, (size_t)nr * row_size, st.d_bad, st.stream);
        if (err == cudaSuccess) err = cudaMemcpyAsync(out + (size_t)r0 * row_size, d_out, (size_t)nr * row_size, cudaMemcpyDeviceToHost, st.stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(st.stream);
        if (err != cudaSuccess) { cudaGetLastError(); return 0; }
        st.collect_violations();
    }
    return staging_ok() ? (size_t)nrows * row_size : 0;
}

extern "C" size_t libgguf_dequantize_chunk(enum ggml_type type, const void *src, float *dst, int64_t start, int64_t nrows,
                                           int64_t n_per_row) {
    if (nrows <= 0 || !src || !dst) return 0;
    const size_t row_size = libgguf_row_size(type, n_per_row);
    if (row_size == 0 || n_per_row <= 0 || start < 0 || start % n_per_row != 0) return 0;
    if (block_geom((int)type).elems == 0) return 0;  // plain storage types have no decoder here (upstream libgguf.cpp:510-586)
    int dev = 0;
    if (!pick_device(&dev) || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return 0; }
    const size_t start_row = (size_t)(start / n_per_row);
    const char *in = (const char *)src + start_row * row_size;
    float *out = dst + start;
    HostCallStaging &st = g_staging[dev];
    std::lock_guard<std::mutex> guard(st.lock);
    if (!st.stream && cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); return 0; }
    const size_t out_row = (size_t)n_per_row * 4;
    if ((size_t)nrows * out_row >= kPipelineBytes && pipeline_enabled()) {
        const int64_t rpp = piece_rows(row_size, out_row, nrows);
        if (!st.ring.reserve((size_t)rpp * row_size, (size_t)rpp * out_row)) { cudaGetLastError(); return 0; }
        const cudaError_t err = run_staged(st.ring, in, row_size, (char *)out, out_row, nrows, rpp,
            [&](const void *d_in, void *d_out, int64_t, int64_t nr, cudaStream_t stream) {
                return launch_dequantize((int)type, d_in, d_out, nr * n_per_row, 0, stream);
            });
        if (err != cudaSuccess) { cudaGetLastError(); return 0; }
        return (size_t)nrows * (size_t)n_per_row * sizeof(float);
    }
    int64_t rows_per_piece = (int64_t)(kStageBytes / out_row);
    if (rows_per_piece < 1) rows_per_piece = 1;
    if (rows_per_piece > nrows) rows_per_piece = nrows;
    if (!grow(&st.d_in, &st.in_cap, (size_t)rows_per_piece * row_size)) return 0;
    if (!grow(&st.d_out, &st.out_cap, (size_t)rows_per_piece * out_row)) return 0;
    if (!st.ensure_counter()) return 0;
    char *d_in = guarded(st.d_in), *d_out = guarded(st.d_out);
    for (int64_t r0 = 0; r0 < nrows; r0 += rows_per_piece) {
        const int64_t nr = nrows - r0 < rows_per_piece ? nrows - r0 : rows_per_piece;
        cudaError_t err = guards_arm(d_in, (size_t)nr * row_size, d_out, (size_t)nr * out_row, st.stream);
        if (err == cudaSuccess) err = cudaMemcpyAsync(d_in, in + (size_t)r0 * row_size, (size_t)nr * row_size, cudaMemcpyHostToDevice, st.stream);
        if (err == cudaSuccess) err = launch_dequantize((int)type, d_in, d_out, nr * n_per_row, 0, st.stream);
        if (err == cudaSuccess) err = guards_check(d_out, (size_t)nr * out_row, st.d_bad, st.stream);
        if (err == cudaSuccess) err = cudaMemcpyAsync(out + r0 * n_per_row, d_out, (size_t)nr * out_row, cudaMemcpyDeviceToHost, st.stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(st.stream);
        if (err != cudaSuccess) { cudaGetLastError(); return 0; }
        st.collect_violations();
    }
    return (size_t)nrows * (size_t)n_per_row * sizeof(float);
}

extern "C" void libgguf_quantize_free(void) {
    int saved = 0;
    const bool have = cudaGetDevice(&saved) == cudaSuccess;
    for (int dev = 0; dev < kMaxDevices; ++dev) {
        HostCallStaging &st = g_staging[dev];
        std::lock_guard<std::mutex> guard(st.lock);
        if (st.d_in || st.d_out || st.d_imatrix || st.stream || st.ring.stream[0]) {
            if (cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); continue; }
            if (st.stream) cudaStreamSynchronize(st.stream);
            st.ring.release();
            cudaFree(st.d_in); cudaFree(st.d_out); cudaFree(st.d_imatrix); cudaFree(st.d_bad);
            st.d_bad = nullptr;
            if (st.stream) cudaStreamDestroy(st.stream);
            st.d_in = st.d_out = nullptr;
            st.d_imatrix = nullptr;
            st.in_cap = st.out_cap = st.im_cap = 0;
            st.stream = nullptr;
        }
    }
    device_state_release_all();
    if (have) cudaSetDevice(saved);
    cudaGetLastError();
}

extern "C" int libgguf_cuda_checked_violations(uint64_t *count) {
    if (!count) return 1;  // LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT
    *count = g_guard_violations.load();
    return checked_mode() ? 0 : 2;  // LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE: the mode is off, nothing was checked
}

// Column sums of squares of a host matrix, staged through the GPU in row pieces (order preserved).
extern "C" int libgguf_cuda_auto_imatrix(const float *host_rows, int64_t rows, int64_t n_per_row, float *host_imatrix) {
    if (rows < 0 || n_per_row <= 0 || !host_imatrix || (rows > 0 && !host_rows)) return 1;  // LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT
    int dev = 0;
    if (!pick_device(&dev) || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return 3; }  // LIBGGUF_CUDA_STATUS_CUDA_ERROR
    HostCallStaging &st = g_staging[dev];
    std::lock_guard<std::mutex> guard(st.lock);
    if (!st.stream && cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); return 3; }
    const size_t row_bytes = (size_t)n_per_row * 4;
    int64_t piece = (int64_t)(kStageBytes / row_bytes);
    if (piece < 1) piece = 1;
    if (piece > rows) piece = rows > 0 ? rows : 1;
    if (!grow(&st.d_in, &st.in_cap, (size_t)piece * row_bytes) || !grow((void **)&st.d_imatrix, &st.im_cap, row_bytes)) return 4;  // ALLOCATION_FAILED
    cudaError_t e = cudaMemsetAsync(st.d_imatrix, 0, row_bytes, st.stream);
    for (int64_t r = 0; r < rows && e == cudaSuccess; r += piece) {
        const int64_t nr = rows - r < piece ? rows - r : piece;
        e = cudaMemcpyAsync(st.d_in, host_rows + r * n_per_row, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, st.stream);
        if (e == cudaSuccess) e = gguf::launch_sumsq_columns((const float *)st.d_in, nr, n_per_row, st.d_imatrix, st.stream);
        // the staging buffer is reused by the next piece: wait for the kernel that reads it
        if (e == cudaSuccess) e = cudaStreamSynchronize(st.stream);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_imatrix, st.d_imatrix, row_bytes, cudaMemcpyDeviceToHost, st.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st.stream);
    if (e != cudaSuccess) { cudaGetLastError(); return 3; }
    return 0;
}
