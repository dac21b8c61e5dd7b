/*
 * Host-pointer C ABI of the GGUF row quantize / dequantize path, B200 build.
 *
 * Every entry point keeps the name, argument order, argument meaning and return convention of
 * the upstream library's public header (upstream include/libgguf.h:102-124), so a program or
 * binding linked against upstream can be relinked against this library unchanged.  All buffers
 * are caller-owned HOST memory; the library moves them to the GPU, runs its sm_100a kernels and
 * moves the result back.  There is no CPU implementation behind these calls: without a usable
 * CUDA device the chunk functions return 0.
 *
 * Numeric values of enum ggml_type are the GGUF wire values (upstream include/libgguf.h:16-61).
 */
#ifndef LIBGGUF_B200_LIBGGUF_H
#define LIBGGUF_B200_LIBGGUF_H

#include <stddef.h>
#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#if defined(_WIN32) && !defined(__MINGW32__)
#define LIBGGUF_API __declspec(dllexport)
#else
#define LIBGGUF_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF tensor type codes.  Gaps are codes the format retired. */
enum ggml_type {
    GGML_TYPE_F32 = 0,
    GGML_TYPE_F16 = 1,
    GGML_TYPE_Q4_0 = 2,
    GGML_TYPE_Q4_1 = 3,
    GGML_TYPE_Q5_0 = 6,
    GGML_TYPE_Q5_1 = 7,
    GGML_TYPE_Q8_0 = 8,
    GGML_TYPE_Q8_1 = 9,
    GGML_TYPE_Q2_K = 10,
    GGML_TYPE_Q3_K = 11,
    GGML_TYPE_Q4_K = 12,
    GGML_TYPE_Q5_K = 13,
    GGML_TYPE_Q6_K = 14,
    GGML_TYPE_Q8_K = 15,
    GGML_TYPE_IQ2_XXS = 16,
    GGML_TYPE_IQ2_XS = 17,
    GGML_TYPE_IQ3_XXS = 18,
    GGML_TYPE_IQ1_S = 19,
    GGML_TYPE_IQ4_NL = 20,
    GGML_TYPE_IQ3_S = 21,
    GGML_TYPE_IQ2_S = 22,
    GGML_TYPE_IQ4_XS = 23,
    GGML_TYPE_I8 = 24,
    GGML_TYPE_I16 = 25,
    GGML_TYPE_I32 = 26,
    GGML_TYPE_I64 = 27,
    GGML_TYPE_F64 = 28,
    GGML_TYPE_IQ1_M = 29,
    GGML_TYPE_BF16 = 30,
    GGML_TYPE_TQ1_0 = 34,
    GGML_TYPE_TQ2_0 = 35,
    GGML_TYPE_MXFP4 = 39,
    GGML_TYPE_NVFP4 = 40,
    GGML_TYPE_Q1_0 = 41,
    GGML_TYPE_COUNT = 42
};

/* Not used by any function below; declared because programs written against the upstream header name
 * them (upstream include/libgguf.h:63-100).  ggml_prec is the precision tag of a tensor operation. */
enum ggml_prec {
    GGML_PREC_DEFAULT = 0,
    GGML_PREC_F32 = 10
};

/* File-level type tag of a model ("general.file_type"): the type most tensors are stored in. */
enum ggml_ftype {
    GGML_FTYPE_UNKNOWN = -1,
    GGML_FTYPE_ALL_F32 = 0,
    GGML_FTYPE_MOSTLY_F16 = 1,
    GGML_FTYPE_MOSTLY_Q4_0 = 2,
    GGML_FTYPE_MOSTLY_Q4_1 = 3,
    GGML_FTYPE_MOSTLY_Q4_1_SOME_F16 = 4,
    GGML_FTYPE_MOSTLY_Q8_0 = 7,
    GGML_FTYPE_MOSTLY_Q5_0 = 8,
    GGML_FTYPE_MOSTLY_Q5_1 = 9,
    GGML_FTYPE_MOSTLY_Q2_K = 10,
    GGML_FTYPE_MOSTLY_Q3_K = 11,
    GGML_FTYPE_MOSTLY_Q4_K = 12,
    GGML_FTYPE_MOSTLY_Q5_K = 13,
    GGML_FTYPE_MOSTLY_Q6_K = 14,
    GGML_FTYPE_MOSTLY_IQ2_XXS = 15,
    GGML_FTYPE_MOSTLY_IQ2_XS = 16,
    GGML_FTYPE_MOSTLY_IQ3_XXS = 17,
    GGML_FTYPE_MOSTLY_IQ1_S = 18,
    GGML_FTYPE_MOSTLY_IQ4_NL = 19,
    GGML_FTYPE_MOSTLY_IQ3_S = 20,
    GGML_FTYPE_MOSTLY_IQ2_S = 21,
    GGML_FTYPE_MOSTLY_IQ4_XS = 22,
    GGML_FTYPE_MOSTLY_IQ1_M = 23,
    GGML_FTYPE_MOSTLY_BF16 = 24,
    GGML_FTYPE_MOSTLY_MXFP4 = 25,
    GGML_FTYPE_MOSTLY_NVFP4 = 26,
    GGML_FTYPE_MOSTLY_Q1_0 = 27
};

/* Bytes of one encoded row of n_per_row elements; 0 if the type has no row encoding or
 * n_per_row is not a positive multiple of the type's block size.
 * Replaces upstream csrc/libgguf.cpp:21-88. */
LIBGGUF_API size_t libgguf_row_size(enum ggml_type type, int64_t n_per_row);

/* Bytes of one encoded block (or one scalar for the plain storage types); 0 if unknown.
 * Replaces upstream csrc/libgguf.cpp:90-164. */
LIBGGUF_API size_t libgguf_type_size(enum ggml_type type);

/* Lower-case GGUF name ("q4_K", "iq2_xxs", ...), "unknown" otherwise.
 * Replaces upstream csrc/libgguf.cpp:166-241. */
LIBGGUF_API const char *libgguf_type_name(enum ggml_type type);

/* True for the types whose quantizer cannot run without importance weights
 * (IQ2_XXS, IQ2_XS, IQ1_S).  Replaces upstream csrc/libgguf.cpp:276-281. */
LIBGGUF_API bool libgguf_quantize_requires_imatrix(enum ggml_type type);

/* Releases the lazily built IQ search tables and the per-device staging buffers.
 * Replaces upstream csrc/libgguf.cpp:265-274. */
LIBGGUF_API void libgguf_quantize_free(void);

/* Quantizes rows [start/n_per_row, start/n_per_row + nrows) of a row-major fp32 matrix.
 *   src      base of the whole matrix (host); the rows read start at src + start
 *   dst      base of the whole encoded matrix (host); rows land at (start/n_per_row)*row_size
 *   start    ELEMENT offset of the first row, a multiple of n_per_row
 *   imatrix  n_per_row importance weights shared by all rows, or NULL
 * Returns the bytes written (nrows * row_size), or 0 on any invalid argument or device error.
 * Replaces upstream csrc/libgguf.cpp:407-484. */
LIBGGUF_API size_t libgguf_quantize_chunk(
    enum ggml_type type,
    const float *src,
    void *dst,
    int64_t start,
    int64_t nrows,
    int64_t n_per_row,
    const float *imatrix);

/* Decodes rows [start/n_per_row, ...) of an encoded matrix to fp32 at dst + start.
 * Returns nrows * n_per_row * 4, or 0 on any invalid argument or device error.
 * Replaces upstream csrc/libgguf.cpp:591-652. */
LIBGGUF_API size_t libgguf_dequantize_chunk(
    enum ggml_type type,
    const void *src,
    float *dst,
    int64_t start,
    int64_t nrows,
    int64_t n_per_row);

#ifdef __cplusplus
}
#endif

#endif /* LIBGGUF_B200_LIBGGUF_H */
