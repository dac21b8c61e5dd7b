// Per-translation-unit copies of the small format tables.  The IQ codebooks are kept packed
// (2 or 3 bits per coordinate); the decoders and the quantizers expand a code with two integer
// instructions instead of loading an expanded 8-byte grid entry.
#pragma once

#include "gguf_common.cuh"

namespace gguf {

// Non-linear 4-bit levels (upstream libgguf_tables.cpp kvalues_iq4nl) and the E2M1 levels times
// two (kvalues_mxfp4).
static GGUF_TABLE int8_t k_iq4nl_values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static GGUF_TABLE int8_t k_fp4_values[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

#define GGUF_CODEBOOK(name, count, ...) static GGUF_TABLE uint16_t k_codebook_##name[count] = {__VA_ARGS__};
#include "gguf_codebooks.inc"
#undef GGUF_CODEBOOK

// Byte value of one coordinate in the expanded decode grids
// (upstream libgguf_tables.cpp iq2xxs_grid/iq2xs_grid/iq2s_grid use {8,25,43}; iq3xxs_grid uses
// 4+8c with 62 for c=7; iq3s_grid uses 2c+1; iq1s_grid uses c-1).
GGUF_HD int iq2_grid_byte(int c) { return 8 + 17 * c + (c >> 1); }
GGUF_HD int iq3xxs_grid_byte(int c) { return 4 + 8 * c + (c == 7 ? 2 : 0); }
GGUF_HD int iq3s_grid_byte(int c) { return 2 * c + 1; }
GGUF_HD int iq1_grid_value(int c) { return c - 1; }

// The 7-bit sign index of the IQ2/IQ3 formats gets an eighth bit that makes the parity even
// (upstream libgguf_tables.cpp ksigns_iq2xs).
GGUF_HD uint32_t iq_signs_from_index(uint32_t i7) {
#ifdef __CUDA_ARCH__
    return i7 | ((uint32_t)(__popc(i7) & 1) << 7);
#else
    return i7 | ((uint32_t)(__builtin_popcount(i7) & 1) << 7);
#endif
}

}  // namespace gguf
