// Device-pointer C ABI (include/libgguf_cuda_native.h): contexts, events, grow-only buffers,
// async copies and the row quantize / dequantize entry points.
#include <math.h>
#include <limits>
#include <new>
#include <string>

#include "../../include/libgguf.h"
#include "../../include/libgguf_cuda_native.h"
#include "device_state.h"
#include "gguf_common.cuh"
#include "host_stage.h"
#include "kernels.h"

struct libgguf_cuda_context {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string last_error;
};
struct libgguf_cuda_buffer {
    void *data = nullptr;
    size_t size = 0;
    size_t capacity = 0;
};
struct libgguf_cuda_host_buffer {
    void *data = nullptr;
    size_t size = 0;
    size_t capacity = 0;
};
struct libgguf_cuda_event {
    cudaEvent_t event = nullptr;
};

using namespace gguf;

namespace gguf {
cudaError_t selftest_fp4(float e, int mode, int ebyte, unsigned long long *device_counters, cudaStream_t stream);
int64_t static_scratch_max_rows();
cudaError_t launch_quantize_legacy_weighted_static(int type, const float *src, const float *qw, void *dst, int64_t nrows,
                                                   int64_t n_per_row, cudaStream_t stream);
}  // namespace gguf

namespace {

thread_local std::string t_thread_error;

int fail(libgguf_cuda_context *ctx, int status, const char *message) {
    if (ctx) ctx->last_error = message ? message : "";
    else t_thread_error = message ? message : "";
    return status;
}
int ok(libgguf_cuda_context *ctx) { return fail(ctx, LIBGGUF_CUDA_STATUS_SUCCESS, ""); }
int cuda_fail(libgguf_cuda_context *ctx, cudaError_t error) {
    cudaGetLastError();  // clear the sticky-free error state
    return fail(ctx, LIBGGUF_CUDA_STATUS_CUDA_ERROR, cudaGetErrorString(error));
}
int use_device(libgguf_cuda_context *ctx) {
    if (!ctx) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    const cudaError_t error = cudaSetDevice(ctx->device);
    return error == cudaSuccess ? LIBGGUF_CUDA_STATUS_SUCCESS : cuda_fail(ctx, error);
}

int64_t decode_block_elems(int64_t qtype) {
    if (qtype == GGML_TYPE_BF16) return 1;
    return block_geom((int)qtype).elems;
}
int64_t decode_row_bytes(int64_t qtype, int64_t n_per_row) {
    if (n_per_row < 0) return 0;
    if (qtype == GGML_TYPE_BF16) {
        if (n_per_row > std::numeric_limits<int64_t>::max() / 2) return 0;
        return n_per_row * 2;
    }
    if (qtype < 0 || qtype >= GGML_TYPE_COUNT || block_geom((int)qtype).elems == 0) return 0;
    return (int64_t)libgguf_row_size((enum ggml_type)qtype, n_per_row);
}

int run_dequantize(libgguf_cuda_context *ctx, const void *device_input, int64_t qtype, int64_t rows, int64_t n_per_row,
                   int output_dtype, void *device_output, cudaStream_t stream) {
    if (!device_input || !device_output || rows < 0 || n_per_row <= 0)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid dequantize arguments");
    if (output_dtype != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F32 && output_dtype != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F16 &&
        output_dtype != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_BF16)
        return fail(ctx, LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE, "unsupported CUDA dequantize output dtype");
    const int64_t block = decode_block_elems(qtype);
    if (block <= 0 || (qtype != GGML_TYPE_BF16 && block_geom((int)qtype).elems == 0))
        return fail(ctx, LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE, "unsupported CUDA dequantization type");
    if (n_per_row % block != 0)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "row width is not divisible by dequantization block size");
    if (rows > std::numeric_limits<int64_t>::max() / 8 / n_per_row)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "dequantize output element count is too large");
    if (rows == 0) return ok(ctx);
    const cudaError_t error = launch_dequantize((int)qtype, device_input, device_output, rows * n_per_row, output_dtype, stream);
    if (error != cudaSuccess) return cuda_fail(ctx, error);
    return ok(ctx);
}

int run_quantize(libgguf_cuda_context *ctx, const float *device_input, const float *device_imatrix, void *device_output,
                 int64_t qtype, int64_t rows, int64_t n_per_row, cudaStream_t stream) {
    if (!device_input || !device_output || rows < 0 || n_per_row <= 0)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid quantize arguments");
    if (qtype < 0 || qtype >= GGML_TYPE_COUNT || !quantize_supported((int)qtype))
        return fail(ctx, LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE, "unsupported CUDA quantization type");
    if (reinterpret_cast<uintptr_t>(device_input) & 15)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "device_input must be 16-byte aligned");
    const int64_t block = block_geom((int)qtype).elems;
    if (n_per_row % block != 0)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "row width is not divisible by quantization block size");
    if (libgguf_quantize_requires_imatrix((enum ggml_type)qtype) && !device_imatrix)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "quantization type requires an imatrix");
    if (rows == 0) return ok(ctx);
    int dev = 0;
    cudaError_t error = cudaGetDevice(&dev);
    if (error != cudaSuccess) return cuda_fail(ctx, error);
    const DeviceState *state = device_state_for((int)qtype, dev);
    if (!state) return fail(ctx, LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED, "failed to build the quantizer tables on the device");
    error = launch_quantize((int)qtype, device_input, device_imatrix, device_output, rows, n_per_row, state, stream);
    if (error != cudaSuccess) return cuda_fail(ctx, error);
    return ok(ctx);
}

template <class B, class AllocFn, class FreeFn>
int resize_discard(libgguf_cuda_context *ctx, B *buffer, size_t size, AllocFn alloc, FreeFn release) {
    if (size <= buffer->capacity) {
        buffer->size = size;
        return ok(ctx);
    }
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    if (buffer->data) {
        const cudaError_t free_error = release(buffer->data);
        buffer->data = nullptr;
        buffer->size = buffer->capacity = 0;
        if (free_error != cudaSuccess) return cuda_fail(ctx, free_error);
    }
    void *data = nullptr;
    const cudaError_t alloc_error = alloc(&data, size);
    if (alloc_error != cudaSuccess) return cuda_fail(ctx, alloc_error);
    buffer->data = data;
    buffer->size = buffer->capacity = size;
    return ok(ctx);
}

}  // namespace

extern "C" {

int libgguf_cuda_context_create(int device, libgguf_cuda_context **out) {
    if (!out) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    *out = nullptr;
    libgguf_cuda_context *ctx = new (std::nothrow) libgguf_cuda_context();
    if (!ctx) return LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED;
    ctx->device = device;
    cudaError_t error = cudaSetDevice(device);
    if (error == cudaSuccess) error = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (error != cudaSuccess) {
        cudaGetLastError();
        delete ctx;
        return LIBGGUF_CUDA_STATUS_CUDA_ERROR;
    }
    *out = ctx;
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

void libgguf_cuda_context_destroy(libgguf_cuda_context *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *libgguf_cuda_last_error(const libgguf_cuda_context *ctx) {
    return ctx ? ctx->last_error.c_str() : "libgguf CUDA context is null";
}

const char *libgguf_cuda_thread_last_error(void) { return t_thread_error.c_str(); }

uint64_t libgguf_cuda_kernel_launch_count(void) { return launch_count(); }

void libgguf_cuda_host_copy(void *dst, const void *src, size_t bytes) {
    if (dst && src && bytes) gguf::parallel_copy(dst, src, bytes);
}

int libgguf_cuda_staging_timeouts(uint64_t *count) {
    if (!count) return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "staging_timeouts requires an output pointer");
    unsigned long long value = 0;
    const cudaError_t error = gguf::read_staging_timeouts(&value);
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    *count = value;
    return ok(nullptr);
}

int libgguf_cuda_set_staging_wait_limit(int limit) {
    const cudaError_t error = gguf::set_staging_wait_limit(limit);
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    return ok(nullptr);
}

int libgguf_cuda_event_create(libgguf_cuda_context *ctx, libgguf_cuda_event **out) {
    if (!ctx || !out) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "event create requires a context and output pointer");
    *out = nullptr;
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    libgguf_cuda_event *event = new (std::nothrow) libgguf_cuda_event();
    if (!event) return fail(ctx, LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED, "failed to allocate CUDA event handle");
    const cudaError_t error = cudaEventCreate(&event->event);
    if (error != cudaSuccess) {
        delete event;
        return cuda_fail(ctx, error);
    }
    *out = event;
    return ok(ctx);
}

void libgguf_cuda_event_destroy(libgguf_cuda_context *ctx, libgguf_cuda_event *event) {
    if (!event) return;
    if (ctx) cudaSetDevice(ctx->device);
    if (event->event) cudaEventDestroy(event->event);
    delete event;
}

int libgguf_cuda_event_record(libgguf_cuda_context *ctx, libgguf_cuda_event *event) {
    if (!ctx || !event) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "event record requires a context and event");
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    const cudaError_t error = cudaEventRecord(event->event, ctx->stream);
    return error == cudaSuccess ? ok(ctx) : cuda_fail(ctx, error);
}

int libgguf_cuda_event_synchronize(libgguf_cuda_context *ctx, libgguf_cuda_event *event) {
    if (!ctx || !event) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "event synchronize requires a context and event");
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    const cudaError_t error = cudaEventSynchronize(event->event);
    return error == cudaSuccess ? ok(ctx) : cuda_fail(ctx, error);
}

int libgguf_cuda_event_elapsed_ms(libgguf_cuda_context *ctx, const libgguf_cuda_event *start, const libgguf_cuda_event *end,
                                  float *out) {
    if (!ctx || !start || !end || !out)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "event elapsed requires a context, two events and an output pointer");
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    const cudaError_t error = cudaEventElapsedTime(out, start->event, end->event);
    return error == cudaSuccess ? ok(ctx) : cuda_fail(ctx, error);
}

int libgguf_cuda_qtype_supported(int64_t qtype) {
    return qtype >= 0 && qtype < GGML_TYPE_COUNT && quantize_supported((int)qtype);
}
int libgguf_cuda_qtype_needs_imatrix(int64_t qtype) {
    return qtype >= 0 && qtype < GGML_TYPE_COUNT && libgguf_quantize_requires_imatrix((enum ggml_type)qtype);
}
int64_t libgguf_cuda_block_size(int64_t qtype) {
    return libgguf_cuda_qtype_supported(qtype) ? block_geom((int)qtype).elems : 0;
}
int64_t libgguf_cuda_row_size(int64_t qtype, int64_t n_per_row) {
    return libgguf_cuda_qtype_supported(qtype) ? (int64_t)libgguf_row_size((enum ggml_type)qtype, n_per_row) : 0;
}
int libgguf_cuda_dequantize_qtype_supported(int64_t qtype) { return decode_block_elems(qtype) > 0; }
int64_t libgguf_cuda_dequantize_block_size(int64_t qtype) { return decode_block_elems(qtype); }
int64_t libgguf_cuda_dequantize_row_size(int64_t qtype, int64_t n_per_row) { return decode_row_bytes(qtype, n_per_row); }

int libgguf_cuda_buffer_create(libgguf_cuda_context *ctx, size_t size, libgguf_cuda_buffer **out) {
    if (!ctx || !out) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "buffer create requires a context and output pointer");
    *out = nullptr;
    libgguf_cuda_buffer *buffer = new (std::nothrow) libgguf_cuda_buffer();
    if (!buffer) return fail(ctx, LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED, "failed to allocate CUDA buffer handle");
    const int status = libgguf_cuda_buffer_resize_discard(ctx, buffer, size);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) {
        delete buffer;
        return status;
    }
    *out = buffer;
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

void libgguf_cuda_buffer_destroy(libgguf_cuda_context *ctx, libgguf_cuda_buffer *buffer) {
    if (!buffer) return;
    if (ctx) cudaSetDevice(ctx->device);
    if (buffer->data) cudaFree(buffer->data);
    delete buffer;
}

int libgguf_cuda_buffer_resize_discard(libgguf_cuda_context *ctx, libgguf_cuda_buffer *buffer, size_t size) {
    if (!ctx || !buffer) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "buffer discard resize requires a context and buffer");
    return resize_discard(ctx, buffer, size, [](void **p, size_t n) { return cudaMalloc(p, n); }, [](void *p) { return cudaFree(p); });
}

void *libgguf_cuda_buffer_data(libgguf_cuda_buffer *buffer) { return buffer ? buffer->data : nullptr; }
const void *libgguf_cuda_buffer_const_data(const libgguf_cuda_buffer *buffer) { return buffer ? buffer->data : nullptr; }
size_t libgguf_cuda_buffer_size(const libgguf_cuda_buffer *buffer) { return buffer ? buffer->size : 0; }

int libgguf_cuda_host_buffer_create(libgguf_cuda_context *ctx, size_t size, libgguf_cuda_host_buffer **out) {
    if (!ctx || !out) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "host buffer create requires a context and output pointer");
    *out = nullptr;
    libgguf_cuda_host_buffer *buffer = new (std::nothrow) libgguf_cuda_host_buffer();
    if (!buffer) return fail(ctx, LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED, "failed to allocate CUDA host buffer handle");
    const int status = libgguf_cuda_host_buffer_resize_discard(ctx, buffer, size);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) {
        delete buffer;
        return status;
    }
    *out = buffer;
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

void libgguf_cuda_host_buffer_destroy(libgguf_cuda_context *ctx, libgguf_cuda_host_buffer *buffer) {
    if (!buffer) return;
    if (ctx) cudaSetDevice(ctx->device);
    if (buffer->data) cudaFreeHost(buffer->data);
    delete buffer;
}

int libgguf_cuda_host_buffer_resize_discard(libgguf_cuda_context *ctx, libgguf_cuda_host_buffer *buffer, size_t size) {
    if (!ctx || !buffer) return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "host buffer discard resize requires a context and buffer");
    return resize_discard(ctx, buffer, size, [](void **p, size_t n) { return cudaMallocHost(p, n); },
                          [](void *p) { return cudaFreeHost(p); });
}

void *libgguf_cuda_host_buffer_data(libgguf_cuda_host_buffer *buffer) { return buffer ? buffer->data : nullptr; }
const void *libgguf_cuda_host_buffer_const_data(const libgguf_cuda_host_buffer *buffer) { return buffer ? buffer->data : nullptr; }
size_t libgguf_cuda_host_buffer_size(const libgguf_cuda_host_buffer *buffer) { return buffer ? buffer->size : 0; }

int libgguf_cuda_h2d(libgguf_cuda_context *ctx, libgguf_cuda_buffer *dst, size_t dst_offset, const void *src, size_t size) {
    if (!ctx || !dst || (!src && size > 0) || dst_offset > dst->size || size > dst->size - dst_offset)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid host-to-device copy arguments");
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS || size == 0) return status;
    const cudaError_t error = cudaMemcpyAsync(static_cast<char *>(dst->data) + dst_offset, src, size, cudaMemcpyHostToDevice, ctx->stream);
    return error == cudaSuccess ? ok(ctx) : cuda_fail(ctx, error);
}

int libgguf_cuda_d2h(libgguf_cuda_context *ctx, void *dst, const libgguf_cuda_buffer *src, size_t src_offset, size_t size) {
    if (!ctx || (!dst && size > 0) || !src || src_offset > src->size || size > src->size - src_offset)
        return fail(ctx, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid device-to-host copy arguments");
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS || size == 0) return status;
    const cudaError_t error = cudaMemcpyAsync(dst, static_cast<const char *>(src->data) + src_offset, size, cudaMemcpyDeviceToHost, ctx->stream);
    return error == cudaSuccess ? ok(ctx) : cuda_fail(ctx, error);
}

int libgguf_cuda_quantize_f32_rows(libgguf_cuda_context *ctx, const float *device_input, const float *device_imatrix,
                                   void *device_output, int64_t qtype, int64_t rows, int64_t n_per_row) {
    if (!ctx) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    return run_quantize(ctx, device_input, device_imatrix, device_output, qtype, rows, n_per_row, ctx->stream);
}

int libgguf_cuda_quantize_f32_rows_on_stream(const float *device_input, const float *device_imatrix, void *device_output,
                                             int64_t qtype, int64_t rows, int64_t n_per_row, void *stream) {
    return run_quantize(nullptr, device_input, device_imatrix, device_output, qtype, rows, n_per_row,
                        reinterpret_cast<cudaStream_t>(stream));
}

int libgguf_cuda_device_count(int *count) {
    if (!count) return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "count must not be null");
    *count = 0;
    const cudaError_t error = cudaGetDeviceCount(count);
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    return ok(nullptr);
}

int libgguf_cuda_accumulate_imatrix_on_stream(const float *device_rows, int64_t rows, int64_t n_per_row, float *device_imatrix,
                                              void *stream) {
    if (rows < 0 || n_per_row <= 0 || !device_imatrix || (rows > 0 && !device_rows))
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid imatrix accumulation arguments");
    const cudaError_t error = launch_sumsq_columns(device_rows, rows, n_per_row, device_imatrix, reinterpret_cast<cudaStream_t>(stream));
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    return ok(nullptr);
}

int libgguf_cuda_widen_on_stream(const void *device_input, int source_dtype, float *device_output, int64_t count, void *stream) {
    if (count < 0 || (count > 0 && (!device_input || !device_output)))
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid widen arguments");
    if (source_dtype != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F16 && source_dtype != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_BF16)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "source dtype must be F16 (1) or BF16 (2)");
    if (reinterpret_cast<uintptr_t>(device_input) & 1 || reinterpret_cast<uintptr_t>(device_output) & 3)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "widen pointers must be aligned to their element size");
    const cudaError_t error = launch_widen(source_dtype, device_input, device_output, count, reinterpret_cast<cudaStream_t>(stream));
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    return ok(nullptr);
}

int libgguf_cuda_quantize_rows_from_on_stream(const void *device_input, int source_dtype, float *device_f32_scratch,
                                              const float *device_imatrix, void *device_output, int64_t qtype, int64_t rows,
                                              int64_t n_per_row, void *stream) {
    if (source_dtype == LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F32)
        return run_quantize(nullptr, static_cast<const float *>(device_input), device_imatrix, device_output, qtype, rows, n_per_row,
                            reinterpret_cast<cudaStream_t>(stream));
    if (rows < 0 || n_per_row <= 0) return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid quantize arguments");
    if (rows > 0 && !device_f32_scratch)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "a 16-bit source needs an fp32 scratch buffer of rows * n_per_row floats");
    if (reinterpret_cast<uintptr_t>(device_f32_scratch) & 15)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "the fp32 scratch buffer must be 16-byte aligned");
    const int status = libgguf_cuda_widen_on_stream(device_input, source_dtype, device_f32_scratch, rows * n_per_row, stream);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    return run_quantize(nullptr, device_f32_scratch, device_imatrix, device_output, qtype, rows, n_per_row,
                        reinterpret_cast<cudaStream_t>(stream));
}

int libgguf_cuda_dequantize_rows(libgguf_cuda_context *ctx, const void *device_input, int64_t qtype, int64_t rows,
                                 int64_t n_per_row, int output_dtype, void *device_output) {
    if (!ctx) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    const int status = use_device(ctx);
    if (status != LIBGGUF_CUDA_STATUS_SUCCESS) return status;
    return run_dequantize(ctx, device_input, qtype, rows, n_per_row, output_dtype, device_output, ctx->stream);
}

int libgguf_cuda_dequantize_rows_on_stream(const void *device_input, int64_t qtype, int64_t rows, int64_t n_per_row,
                                           int output_dtype, void *device_output, void *stream) {
    return run_dequantize(nullptr, device_input, qtype, rows, n_per_row, output_dtype, device_output,
                          reinterpret_cast<cudaStream_t>(stream));
}

int64_t libgguf_cuda_quantize_weighted_rows_static_max_rows(void) { return static_scratch_max_rows(); }

int libgguf_cuda_quantize_weighted_rows_static(const float *device_input, const float *device_imatrix, void *device_output,
                                               int64_t qtype, int64_t rows, int64_t n_per_row, void *stream) {
    if (!device_input || !device_imatrix || !device_output || rows < 0 || n_per_row <= 0)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "invalid quantize arguments (input, imatrix and output are all required)");
    if (qtype != GGML_TYPE_Q4_0 && qtype != GGML_TYPE_Q4_1 && qtype != GGML_TYPE_Q5_0 && qtype != GGML_TYPE_Q5_1)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE,
                    "the allocation-free entry point covers the importance-weighted Q4_0, Q4_1, Q5_0 and Q5_1 quantizers only");
    if (n_per_row % 32 != 0)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "row width is not divisible by quantization block size");
    if (reinterpret_cast<uintptr_t>(device_input) & 15)
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "device_input must be 16-byte aligned");
    if (rows > static_scratch_max_rows())
        return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT,
                    "too many rows for the built-in scratch array (limit 65536 rows per call): split the call by rows");
    if (rows == 0) return ok(nullptr);
    const cudaError_t error = launch_quantize_legacy_weighted_static((int)qtype, device_input, device_imatrix, device_output, rows,
                                                                     n_per_row, reinterpret_cast<cudaStream_t>(stream));
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    return ok(nullptr);
}

int libgguf_cuda_selftest_fp4_mode(float scale, int mode, uint64_t *mismatches, uint64_t *fallbacks) {
    if (!mismatches) return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "mismatches must not be null");
    if (mode < 0 || mode > 2) return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "mode must be 0, 1 or 2");
    int ebyte = 0;
    if (mode == 1) {
        int exponent = 0;
        const bool power_of_two = scale > 0.f && frexpf(scale, &exponent) == 0.5f;
        ebyte = exponent - 1 + 128;  // scale = 0.5 * 2^exponent
        if (!power_of_two || ebyte > 252 || ebyte < 0)
            return fail(nullptr, LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT, "mode 1 needs a power-of-two scale 2^(e-128), e <= 252");
    }
    unsigned long long *counters = nullptr;
    cudaError_t error = cudaMalloc((void **)&counters, 2 * sizeof(unsigned long long));
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    error = cudaMemset(counters, 0, 2 * sizeof(unsigned long long));
    if (error == cudaSuccess) error = selftest_fp4(scale, mode, ebyte, counters, nullptr);
    unsigned long long host[2] = {0, 0};
    if (error == cudaSuccess) error = cudaMemcpy(host, counters, sizeof(host), cudaMemcpyDeviceToHost);
    cudaFree(counters);
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    *mismatches = host[0];
    if (fallbacks) *fallbacks = host[1];
    return ok(nullptr);
}

int libgguf_cuda_selftest_fp4(float scale, uint64_t *mismatches) { return libgguf_cuda_selftest_fp4_mode(scale, 0, mismatches, nullptr); }

int libgguf_cuda_prepare_qtype(int64_t qtype) {
    if (qtype < 0 || qtype >= GGML_TYPE_COUNT) return fail(nullptr, LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE, "unsupported type");
    int dev = 0;
    const cudaError_t error = cudaGetDevice(&dev);
    if (error != cudaSuccess) return cuda_fail(nullptr, error);
    return device_state_for((int)qtype, dev) ? LIBGGUF_CUDA_STATUS_SUCCESS
                                            : fail(nullptr, LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED, "table upload failed");
}

}  // extern "C"
