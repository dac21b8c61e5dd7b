// Per-device read-only tables the quantizers need: the MXFP4 exponent steps measured from the
// host libm, and the IQ search tables (grid, lattice-point map, neighbour lists).  Built on the
// host once per process, uploaded once per device on first use, released by
// libgguf_quantize_free().
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gguf {

constexpr int kMaxDevices = 64;
constexpr int kIqStepEntries = 4;
enum IqTableId { IQT_2XXS = 0, IQT_2XS, IQT_1S, IQT_2S, IQT_3XXS, IQT_3S, IQT_COUNT };
// shared memory a kernel has for neighbour records beside its codebook and per-warp state (quant_iq23.cu), bytes:
// IQ2_XXS stages none (its 128 registers and 12.5 KB per warp leave 23 KB, and fewer warps cost more than that buys),
// IQ2_XS 84 KB (about 80 % of the reads on Student-t data, 70 % on normal data), IQ2_S 76 KB (97 % / 95 %), IQ3 everything
constexpr int kIqHotBudget[IQT_COUNT] = {0, 86016, 0, 77824, 1 << 20, 1 << 20};

// One IQ codebook prepared for searching (device pointers).
struct IqSearchTable {
    const uint8_t *grid = nullptr;         // grid_size x dims bytes, coordinate value 2*code+1
    const int32_t *map = nullptr;          // lattice index -> grid index (>= 0) or -(offset+1) into neighbours
    const uint16_t *neighbours = nullptr;  // [count, idx0, idx1, ...] runs
    // The neighbour lists again, laid out for the IQ2 / IQ3 scans: every list padded to whole records of record_steps
    // steps of kIqStepEntries entries with copies of its first entry (a copy's distance equals the first entry's, so
    // it is never a strict improvement), records aligned to their size (8 or 16 bytes), an entry stored as the byte
    // offset of its codebook row in the kernel's staged codebook (grid index x dims x 2).  map_s is map with a list's
    // first record and record count folded in: -(((first_record << 8) | records) + 1).  Absent for the IQ1 codebook.
    // Where a kernel can keep only part of the array in shared memory (IQ2) the lists are ordered by how often their
    // lattice point comes up (sum of its levels, ascending: blocks scaled to their maximum are mostly small levels), so
    // a prefix holds most of the scans' reads: hot_bytes = the whole lists at the front that fit kIqHotBudget (0: none
    // staged; records_bytes: all of it, the IQ3 codebooks).
    const void *records = nullptr;
    const int32_t *map_s = nullptr;
    int record_steps = 0;
    int records_bytes = 0;
    int grid_size = 0;
    int dims = 0;
    int map_size = 0;
    int neighbours_len = 0;
    int hot_bytes = 0;
};

struct DeviceState {
    int device = -1;
    const float *mx_steps = nullptr;  // 277 floats, see quant_simple.cu
    IqSearchTable iq[IQT_COUNT];
};

// Returns the state of device `dev` with everything quantizing `type` needs present, building
// and uploading on first use (blocking).  The caller must have made `dev` current.  nullptr on
// allocation or copy failure.
const DeviceState *device_state_for(int type, int dev);

void device_state_release_all();

cudaError_t launch_store(int type, const float *src, void *dst, int64_t nelems, cudaStream_t stream);
cudaError_t launch_quantize(int type, const float *src, const float *imatrix, void *dst, int64_t nrows,
                            int64_t n_per_row, const DeviceState *state, cudaStream_t stream);

}  // namespace gguf
