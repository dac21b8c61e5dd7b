/*
 * Device-pointer C ABI of the GGUF row quantize / dequantize path, B200 build.
 *
 * The first group of functions keeps the names, argument order and status codes of upstream's
 * native CUDA interface (upstream src/libgguf/libgguf_cuda/csrc/libgguf_cuda_native.h:10-107),
 * which is what the upstream converter (csrc/quantize_gguf.cpp:1732-1931) and the upstream
 * ctypes test bind.  Inputs and outputs of the row functions are DEVICE pointers.  All work is
 * asynchronous on the context's stream (or the caller's stream for the *_on_stream variants);
 * only libgguf_cuda_event_synchronize blocks.
 *
 * The second group ("additions") has no upstream counterpart; each is marked.
 */
#ifndef LIBGGUF_B200_CUDA_NATIVE_H
#define LIBGGUF_B200_CUDA_NATIVE_H

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32) && !defined(__MINGW32__)
#define LIBGGUF_CUDA_API __declspec(dllexport)
#else
#define LIBGGUF_CUDA_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* upstream libgguf_cuda_native.h:10-16 */
enum libgguf_cuda_status {
    LIBGGUF_CUDA_STATUS_SUCCESS = 0,
    LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT = 1,
    LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE = 2,
    LIBGGUF_CUDA_STATUS_CUDA_ERROR = 3,
    LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED = 4
};

/* upstream libgguf_cuda_native.h:18-21 has F32 and F16; BF16 is an addition. */
enum libgguf_cuda_dequantize_dtype {
    LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F32 = 0,
    LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F16 = 1,
    LIBGGUF_CUDA_DEQUANTIZE_DTYPE_BF16 = 2
};

typedef struct libgguf_cuda_context libgguf_cuda_context;
typedef struct libgguf_cuda_buffer libgguf_cuda_buffer;
typedef struct libgguf_cuda_event libgguf_cuda_event;
typedef struct libgguf_cuda_host_buffer libgguf_cuda_host_buffer;

/* ---- context, events (upstream libgguf_cuda_native.h:28-41) ---- */
LIBGGUF_CUDA_API int libgguf_cuda_context_create(int device, libgguf_cuda_context **out);
LIBGGUF_CUDA_API void libgguf_cuda_context_destroy(libgguf_cuda_context *ctx);
LIBGGUF_CUDA_API const char *libgguf_cuda_last_error(const libgguf_cuda_context *ctx);
LIBGGUF_CUDA_API int libgguf_cuda_event_create(libgguf_cuda_context *ctx, libgguf_cuda_event **out);
LIBGGUF_CUDA_API void libgguf_cuda_event_destroy(libgguf_cuda_context *ctx, libgguf_cuda_event *event);
LIBGGUF_CUDA_API int libgguf_cuda_event_record(libgguf_cuda_context *ctx, libgguf_cuda_event *event);
LIBGGUF_CUDA_API int libgguf_cuda_event_synchronize(libgguf_cuda_context *ctx, libgguf_cuda_event *event);
LIBGGUF_CUDA_API int libgguf_cuda_event_elapsed_ms(libgguf_cuda_context *ctx, const libgguf_cuda_event *start,
                                                   const libgguf_cuda_event *end, float *out);

/* ---- type queries (upstream libgguf_cuda_native.h:43-49) ---- */
LIBGGUF_CUDA_API int libgguf_cuda_qtype_supported(int64_t qtype);
LIBGGUF_CUDA_API int libgguf_cuda_qtype_needs_imatrix(int64_t qtype);
LIBGGUF_CUDA_API int64_t libgguf_cuda_block_size(int64_t qtype);
LIBGGUF_CUDA_API int64_t libgguf_cuda_row_size(int64_t qtype, int64_t n_per_row);
LIBGGUF_CUDA_API int libgguf_cuda_dequantize_qtype_supported(int64_t qtype);
LIBGGUF_CUDA_API int64_t libgguf_cuda_dequantize_block_size(int64_t qtype);
LIBGGUF_CUDA_API int64_t libgguf_cuda_dequantize_row_size(int64_t qtype, int64_t n_per_row);

/* ---- device and pinned-host buffers, grow-only (upstream libgguf_cuda_native.h:51-63) ---- */
LIBGGUF_CUDA_API int libgguf_cuda_buffer_create(libgguf_cuda_context *ctx, size_t size, libgguf_cuda_buffer **out);
LIBGGUF_CUDA_API void libgguf_cuda_buffer_destroy(libgguf_cuda_context *ctx, libgguf_cuda_buffer *buffer);
LIBGGUF_CUDA_API int libgguf_cuda_buffer_resize_discard(libgguf_cuda_context *ctx, libgguf_cuda_buffer *buffer, size_t size);
LIBGGUF_CUDA_API void *libgguf_cuda_buffer_data(libgguf_cuda_buffer *buffer);
LIBGGUF_CUDA_API const void *libgguf_cuda_buffer_const_data(const libgguf_cuda_buffer *buffer);
LIBGGUF_CUDA_API size_t libgguf_cuda_buffer_size(const libgguf_cuda_buffer *buffer);

LIBGGUF_CUDA_API int libgguf_cuda_host_buffer_create(libgguf_cuda_context *ctx, size_t size, libgguf_cuda_host_buffer **out);
LIBGGUF_CUDA_API void libgguf_cuda_host_buffer_destroy(libgguf_cuda_context *ctx, libgguf_cuda_host_buffer *buffer);
LIBGGUF_CUDA_API int libgguf_cuda_host_buffer_resize_discard(libgguf_cuda_context *ctx, libgguf_cuda_host_buffer *buffer, size_t size);
LIBGGUF_CUDA_API void *libgguf_cuda_host_buffer_data(libgguf_cuda_host_buffer *buffer);
LIBGGUF_CUDA_API const void *libgguf_cuda_host_buffer_const_data(const libgguf_cuda_host_buffer *buffer);
LIBGGUF_CUDA_API size_t libgguf_cuda_host_buffer_size(const libgguf_cuda_host_buffer *buffer);

/* ---- async copies on the context stream (upstream libgguf_cuda_native.h:65-78) ---- */
LIBGGUF_CUDA_API int libgguf_cuda_h2d(libgguf_cuda_context *ctx, libgguf_cuda_buffer *dst, size_t dst_offset,
                                      const void *src, size_t size);
LIBGGUF_CUDA_API int libgguf_cuda_d2h(libgguf_cuda_context *ctx, void *dst, const libgguf_cuda_buffer *src,
                                      size_t src_offset, size_t size);

/* ---- the hot path (upstream libgguf_cuda_native.h:80-105) ----
 * device_imatrix may be NULL unless the type requires importance weights.  Unlike upstream's
 * kernels, a non-NULL imatrix is honoured for every type whose CPU quantizer honours it. */
LIBGGUF_CUDA_API int libgguf_cuda_quantize_f32_rows(libgguf_cuda_context *ctx, const float *device_input,
                                                    const float *device_imatrix, void *device_output,
                                                    int64_t qtype, int64_t rows, int64_t n_per_row);
LIBGGUF_CUDA_API int libgguf_cuda_dequantize_rows(libgguf_cuda_context *ctx, const void *device_input, int64_t qtype,
                                                  int64_t rows, int64_t n_per_row, int output_dtype,
                                                  void *device_output);
LIBGGUF_CUDA_API int libgguf_cuda_dequantize_rows_on_stream(const void *device_input, int64_t qtype, int64_t rows,
                                                            int64_t n_per_row, int output_dtype,
                                                            void *device_output, void *stream);

/* ================= additions (no upstream counterpart) ================= */

/* Same as libgguf_cuda_quantize_f32_rows but on the caller's stream (a cudaStream_t passed as
 * void*) of the current device, without a context; this is what a framework binding that
 * launches on "the current stream" needs.  Returns a libgguf_cuda_status. */
LIBGGUF_CUDA_API int libgguf_cuda_quantize_f32_rows_on_stream(const float *device_input, const float *device_imatrix,
                                                              void *device_output, int64_t qtype, int64_t rows,
                                                              int64_t n_per_row, void *stream);

/* Message of the last failing context-less call on this thread ("" if none). */
LIBGGUF_CUDA_API const char *libgguf_cuda_thread_last_error(void);

/* Number of kernels this library has launched in this process (all devices, all threads). */
LIBGGUF_CUDA_API uint64_t libgguf_cuda_kernel_launch_count(void);

/* No upstream counterpart.  The quantizers that stage their input with bulk asynchronous copies (TQ1_0, TQ2_0, Q1_0)
 * bound every wait for a copy; a wait that runs out makes the CTA count it, wait once more (bounded) for the copies it
 * still has in flight and return: its part of the output is then NOT written.  Stores the count of such events on the
 * current device since the library was loaded; 0 on a healthy device.  Blocking (waits for the device).
 * The calls of this library that synchronise by themselves -- libgguf_quantize_chunk and the conversion pipeline --
 * read the counter around their own work and report failure (0 bytes / the shard is redone on another GPU, or the
 * batch fails) when it moved.  A caller of the asynchronous row functions checks it after its own synchronisation. */
LIBGGUF_CUDA_API int libgguf_cuda_staging_timeouts(uint64_t *count);

/* Checked mode, no upstream counterpart.  With LIBGGUF_B200_CHECKED=1 in the environment when the library is loaded,
 * libgguf_quantize_chunk and libgguf_dequantize_chunk run every piece on the single-buffer path with 4 KiB guard bands
 * directly before and after the device bytes a kernel may write (filled with a pattern before the launch, compared
 * after it) and a band of 0xFF bytes directly after the device input (a read past the end then changes the result).
 * Stores the number of guard bytes found changed since the library was loaded; returns LIBGGUF_CUDA_STATUS_SUCCESS
 * when the mode is on and LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE (count 0) when it is off.  Nothing traps: it is the
 * substitute for a memory checker where none can be run, used by the tests on ragged shapes. */
LIBGGUF_CUDA_API int libgguf_cuda_checked_violations(uint64_t *count);

/* Test hook, no upstream counterpart: the number of polling rounds a consumer of a staged tile spends before it gives
 * up, on the current device.  0 makes every consumer give up at once although its copy is on its way (the kernel then
 * takes the give-up path: count, drain, return), which is how the tests exercise the failure reporting without
 * losing a copy; a negative value restores the default.  Blocking. */
LIBGGUF_CUDA_API int libgguf_cuda_set_staging_wait_limit(int limit);

/* No upstream counterpart.  memcpy split over the library's pool of host copy threads (LIBGGUF_CUDA_COPY_THREADS,
 * default 8 on hosts with 16 or more CPUs); the host-pointer chunk functions of libgguf.h use it to fill and drain
 * their pinned staging slots.  Needs no device.  The ranges must not overlap. */
LIBGGUF_CUDA_API void libgguf_cuda_host_copy(void *dst, const void *src, size_t bytes);

/* Builds (once per device) the IQ search tables a quantizer of this type needs, on the current
 * device, and waits for the upload.  Optional: the row functions do it on first use. */
LIBGGUF_CUDA_API int libgguf_cuda_prepare_qtype(int64_t qtype);

/* Inspection, no upstream counterpart in the ABI: the host copy of the search tables the quantizer of an IQ1 / IQ2 / IQ3
 * type uses (the same data upstream builds into iq2_data / iq3_data, csrc/common/libgguf_iq_tables.cpp:36-417,
 * :487-666).  grid: grid_size x dims coordinate bytes (2 * code + 1); map: lattice index -> grid index, or
 * -(offset + 1) where neighbours[offset] is a count followed by that many grid indices ordered by (distance, index).
 * The pointers stay valid for the life of the process.  Needs no device; any out pointer may be NULL. */
LIBGGUF_CUDA_API int libgguf_cuda_iq_search_table(int64_t qtype, int32_t *grid_size, int32_t *dims, const uint8_t **grid,
                                                  const int32_t **map, int64_t *map_size, const uint16_t **neighbours,
                                                  int64_t *neighbours_len);

/* Inspection, no upstream counterpart: the same neighbour lists in the layout the IQ2 / IQ3 quantizers scan.  Every list
 * is a whole number of records of `record_entries` 16-bit entries (4 or 8), its tail filled with copies of its first
 * entry; an entry is grid index * dims * 2 (the byte offset of the codebook row as the kernel stages it).  map_s is
 * `map` with a list's first record and record count folded in: -(((first_record << 8) | records) + 1).
 * (IQ1: 16 x the grid index.)  Needs no device. */
LIBGGUF_CUDA_API int libgguf_cuda_iq_scan_records(int64_t qtype, int32_t *record_entries, const uint16_t **entries,
                                                  int64_t *entries_len, const int32_t **map_s, int64_t *map_size);

/* Self-test, no upstream counterpart: the MXFP4 / NVFP4 quantizers pick each element's level by threshold
 * comparisons instead of upstream's 16-way scan (libgguf_common.h:321-335).  This runs both on every one of the
 * 2^32 float bit patterns at block scale `scale` on the current device (about a second) and stores how many
 * inputs disagree (the quantizers rely on it being 0).  Blocking. */
LIBGGUF_CUDA_API int libgguf_cuda_selftest_fp4(float scale, uint64_t *mismatches);
/* Same, for the forms the quantizers actually run.  mode 0: as above.  mode 1: the MXFP4 form, built on the hardware
 * E2M1 conversion (`scale` must be 2^(e-128) with integer 0 <= e <= 252).  mode 2: the NVFP4 form, two hardware
 * conversions bracketing the quotient; inputs whose two conversions differ (a tie lies within 2^-21 of the quotient)
 * are settled by one comparison with the midpoint of the two candidate levels, as in the quantizer, and are counted in
 * `fallbacks` (may be null).  Modes 1 and 2 look only at the inputs the quantizers route there (finite, |x| <= 2^20 * scale). */
LIBGGUF_CUDA_API int libgguf_cuda_selftest_fp4_mode(float scale, int mode, uint64_t *mismatches, uint64_t *fallbacks);

/* Number of CUDA devices visible to the process (no upstream counterpart; the converter front end uses it to
 * default to all GPUs). */
LIBGGUF_CUDA_API int libgguf_cuda_device_count(int *count);

/* Device-side source decode, no upstream counterpart (upstream widens 16-bit checkpoints on the CPU before the upload:
 * csrc/quantize_gguf.cpp:1415-1442, :2106-2112).  `source_dtype` uses the LIBGGUF_CUDA_DEQUANTIZE_DTYPE_* codes:
 * F16 or BF16 values are widened to fp32 exactly as the host code does (bf16: 16-bit shift; fp16: exact conversion).
 * libgguf_cuda_quantize_rows_from_on_stream widens into `device_f32_scratch` (rows * n_per_row floats, 16-byte
 * aligned; unused and may be NULL for an F32 source) and then quantizes like libgguf_cuda_quantize_f32_rows_on_stream. */
LIBGGUF_CUDA_API int libgguf_cuda_widen_on_stream(const void *device_input, int source_dtype, float *device_output, int64_t count,
                                                  void *stream);
LIBGGUF_CUDA_API int libgguf_cuda_quantize_rows_from_on_stream(const void *device_input, int source_dtype, float *device_f32_scratch,
                                                               const float *device_imatrix, void *device_output, int64_t qtype,
                                                               int64_t rows, int64_t n_per_row, void *stream);

/* The importance weights upstream derives from the data when a type requires them and the caller has none
 * (csrc/_libgguf_module.cpp:1210-1242 compute_auto_imatrix; src/libgguf/__init__.py:186-189): for every column the sum of
 * squares over the rows, added in row order in fp32.  device_imatrix[c] += sum_r rows[r][c]^2, so a matrix may be fed in
 * row pieces in order, the first onto zeros.  libgguf_cuda_auto_imatrix does this for a host matrix (staged through the
 * GPU selected like for the host-pointer chunk functions) and writes n_per_row floats; returns a libgguf_cuda_status. */
LIBGGUF_CUDA_API int libgguf_cuda_accumulate_imatrix_on_stream(const float *device_rows, int64_t rows, int64_t n_per_row,
                                                               float *device_imatrix, void *stream);
LIBGGUF_CUDA_API int libgguf_cuda_auto_imatrix(const float *host_rows, int64_t rows, int64_t n_per_row, float *host_imatrix);
/* The same for a host matrix of F32, F16 or BF16 values (LIBGGUF_CUDA_DEQUANTIZE_DTYPE_* codes; 16-bit values cross the
 * host link as they are and are widened on the GPU).  A caller that quantizes one tensor in several row pieces -- the
 * converter front end, or one process per GPU each taking a row range -- calls this once for the WHOLE tensor and passes
 * the result as the imatrix of every piece, so that the encoded bytes do not depend on how the tensor was cut. */
LIBGGUF_CUDA_API int libgguf_cuda_auto_imatrix_typed(const void *host_rows, int source_dtype, int64_t rows, int64_t n_per_row,
                                                     float *host_imatrix);

/* ---- multi-GPU streaming conversion (replaces the single-GPU two-slot loop of upstream's converter,
 * csrc/quantize_gguf.cpp:1732-1931 and :2072-2146; the pool itself has no upstream counterpart) ----
 * A batch of tensors (host memory, fp32 rows in, encoded rows out) is cut into shards of whole rows of at most
 * chunk_bytes of input, and the shards are streamed through `slots` in-flight copies per GPU on every listed GPU.
 * Pinned host memory is copied from / to directly, pageable memory through pinned staging.  No GPU talks to
 * another GPU.  libgguf_cuda_pipeline_quantize blocks until the batch is done; the output bytes are independent
 * of the number of GPUs, the chunk size and the order in which shards complete. */
typedef struct libgguf_cuda_pipeline libgguf_cuda_pipeline;
typedef struct libgguf_cuda_tensor_desc {
    int64_t qtype;
    const float *src;     /* rows x n_per_row fp32, host */
    const float *imatrix; /* n_per_row floats (host) or NULL */
    void *dst;            /* rows x row_size bytes, host */
    int64_t rows;
    int64_t n_per_row;
} libgguf_cuda_tensor_desc;
typedef struct libgguf_cuda_shard {
    int32_t tensor;
    int64_t row0;
    int64_t rows;
} libgguf_cuda_shard;
/* slots <= 0 -> 3, chunk_bytes == 0 -> 128 MiB */
LIBGGUF_CUDA_API int libgguf_cuda_pipeline_create(const int *devices, int n_devices, int slots, size_t chunk_bytes,
                                                  libgguf_cuda_pipeline **out);
LIBGGUF_CUDA_API void libgguf_cuda_pipeline_destroy(libgguf_cuda_pipeline *pipe);
LIBGGUF_CUDA_API const char *libgguf_cuda_pipeline_last_error(const libgguf_cuda_pipeline *pipe);
LIBGGUF_CUDA_API int libgguf_cuda_pipeline_quantize(libgguf_cuda_pipeline *pipe, const libgguf_cuda_tensor_desc *tensors,
                                                    int n_tensors);
/* Same with a source dtype per tensor (LIBGGUF_CUDA_DEQUANTIZE_DTYPE_* codes; NULL = all F32): `src` of a tensor with
 * dtype F16 / BF16 points at rows x n_per_row 16-bit values, which cross the host link as they are and are widened
 * on the GPU.  A shard is then at most chunk_bytes of source bytes. */
LIBGGUF_CUDA_API int libgguf_cuda_pipeline_quantize_typed(libgguf_cuda_pipeline *pipe, const libgguf_cuda_tensor_desc *tensors,
                                                          const int32_t *source_dtypes, int n_tensors);
LIBGGUF_CUDA_API int64_t libgguf_cuda_pipeline_plan_typed(const libgguf_cuda_tensor_desc *tensors, const int32_t *source_dtypes,
                                                          int n_tensors, size_t chunk_bytes, libgguf_cuda_shard *out, int64_t max_out);
/* The shard list the pipeline would use (largest first); returns the shard count, -1 on a bad descriptor.
 * Needs no GPU. */
LIBGGUF_CUDA_API int64_t libgguf_cuda_pipeline_plan(const libgguf_cuda_tensor_desc *tensors, int n_tensors, size_t chunk_bytes,
                                                    libgguf_cuda_shard *out, int64_t max_out);
/* Shards completed and seconds spent by each GPU worker in the last batch, and how many shards were handed back. */
LIBGGUF_CUDA_API int libgguf_cuda_pipeline_stats(const libgguf_cuda_pipeline *pipe, int64_t *shards_per_device,
                                                 double *seconds_per_device, int64_t *requeued);
/* Test hook, host side only: the worker of devices[device_slot] reports a failure once it has completed
 * after_shards shards (-1 = never); its unfinished shards go back to the queue for the other GPUs. */
LIBGGUF_CUDA_API int libgguf_cuda_pipeline_inject_failure(libgguf_cuda_pipeline *pipe, int device_slot, int64_t after_shards);

/* Importance-weighted Q4_0 / Q4_1 / Q5_0 / Q5_1 quantization that allocates nothing.  It has no
 * counterpart in upstream.  It exists for callers that are not allowed to allocate device memory
 * at the moment they quantize: a host that owns all GPU memory through its own pool and rejects
 * outside allocations, a process pinned to a fixed memory budget, or a latency-critical loop in
 * which an allocator call is not acceptable.  libgguf_cuda_quantize_f32_rows[_on_stream] obtains
 * one float of scratch per row from the stream-ordered allocator for these types; this entry
 * point keeps that scratch in a fixed array inside the library instead (256 KiB, present on every
 * GPU that loads the library, for the life of the process) and calls no cudaMalloc, cudaFree or
 * other allocating routine.
 *   - device_imatrix is required (n_per_row floats); qtype must be one of the four types above.
 *   - rows may be at most libgguf_cuda_quantize_weighted_rows_static_max_rows() (65536); larger
 *     requests are refused with LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT and a message -- split them.
 *   - The first call on a device looks up the array's device address (once per device, with that
 *     device current); make that first call before starting any stream capture.
 *   - All calls share the one array, which keeps whatever the previous call left in it.  Each
 *     call writes the entries it needs before it reads them, so no clearing is needed, but calls
 *     whose kernels can overlap on the GPU (other streams, other host threads) would race on it:
 *     serialise them.
 * Output bytes are identical to those of libgguf_cuda_quantize_f32_rows_on_stream.
 * Runs asynchronously on `stream` (a cudaStream_t passed as void*) of the current device and
 * returns a libgguf_cuda_status; the message is read with libgguf_cuda_thread_last_error(). */
LIBGGUF_CUDA_API int libgguf_cuda_quantize_weighted_rows_static(const float *device_input, const float *device_imatrix,
                                                                void *device_output, int64_t qtype, int64_t rows,
                                                                int64_t n_per_row, void *stream);
LIBGGUF_CUDA_API int64_t libgguf_cuda_quantize_weighted_rows_static_max_rows(void);

#ifdef __cplusplus
}
#endif

#endif /* LIBGGUF_B200_CUDA_NATIVE_H */
