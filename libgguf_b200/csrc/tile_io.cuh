// Coalesced write-out of a CTA's encoded tile.
//
// Quantizers assemble their packed blocks in shared memory (block sizes such as 34 or 110 bytes
// cannot be written with aligned vector stores one block at a time).  The tile is placed in
// shared memory at the same offset modulo 16 as its destination in global memory, so the
// 16-byte aligned middle part moves as uint4 vectors and only the ragged head and tail (at most
// 15 bytes each) move as single bytes -- those bytes may share a 16-byte granule with a
// neighbouring CTA's tile and must not be overwritten.
#pragma once

#include "gguf_common.cuh"

namespace gguf {

// smem_tile must satisfy (smem_tile & 15) == (gdst & 15).
GGUF_D void flush_tile(const uint8_t *smem_tile, uint8_t *gdst, int nbytes, int tid, int nthreads) {
    const int mis = (int)(reinterpret_cast<uintptr_t>(gdst) & 15);
    int head = mis ? 16 - mis : 0;
    if (head > nbytes) head = nbytes;
    const int nvec = (nbytes - head) >> 4;
    const int tail_begin = head + (nvec << 4);
    if (tid < head) gdst[tid] = smem_tile[tid];
    const uint4 *s16 = reinterpret_cast<const uint4 *>(smem_tile + head);
    uint4 *g16 = reinterpret_cast<uint4 *>(gdst + head);
    for (int i = tid; i < nvec; i += nthreads) __stcs(g16 + i, s16[i]);
    const int ntail = nbytes - tail_begin;
    if (tid < ntail) gdst[tail_begin + tid] = smem_tile[tail_begin + tid];
}

}  // namespace gguf
