/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Plain-C, single-threaded restatement of the upstream CPU REF algorithms for the GGUF row
 * quantize / dequantize path.  It exists so that the CUDA kernels can be checked on machines
 * where the upstream sources are not present.  Only tests/, __graft_entry__.smoke() and the
 * cpu_baseline / reference legs of bench.py may load it.
 *
 * Parity pin: tests/test_oracle_golden.py checks every function here against upstream's 70
 * frozen SHA-256 vectors (tests/golden/upstream_manifest.json), against the fixtures generated
 * by running the upstream REF backend (tests/golden/golden.json), and, when oracle/_ref is
 * built, byte-for-byte against the upstream library on random rows.
 *
 * Must be compiled without FMA contraction and without fast-math (see oracle/Makefile).
 */
#ifndef GGUF_ORACLE_H
#define GGUF_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

size_t gguf_oracle_row_size(int type, int64_t n_per_row);
int gguf_oracle_quantize_requires_imatrix(int type);
/* 1 if gguf_oracle_quantize_chunk implements this type (all decoders are implemented). */
int gguf_oracle_quantize_supported(int type);
/* Same contracts as libgguf_quantize_chunk / libgguf_dequantize_chunk (upstream
 * csrc/libgguf.cpp:311-405 and :486-589), single-threaded. */
size_t gguf_oracle_quantize_chunk(int type, const float *src, void *dst, int64_t start, int64_t nrows,
                                  int64_t n_per_row, const float *imatrix);
size_t gguf_oracle_dequantize_chunk(int type, const void *src, float *dst, int64_t start, int64_t nrows,
                                    int64_t n_per_row);

#ifdef __cplusplus
}
#endif
#endif
