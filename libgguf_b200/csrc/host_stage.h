// Staging of the host-pointer calls: pageable caller memory <-> pinned ring <-> device, pipelined.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <functional>

namespace gguf {

// memcpy split over a small pool of worker threads (the calling thread takes a share).  One copy at a time.
void parallel_copy(void *dst, const void *src, size_t bytes);

// Two slots of pinned host and device memory for each direction, two streams, grow-only.
struct StageRing {
    void *h_in[2] = {nullptr, nullptr}, *h_out[2] = {nullptr, nullptr};
    void *d_in[2] = {nullptr, nullptr}, *d_out[2] = {nullptr, nullptr};
    size_t in_cap = 0, out_cap = 0;
    cudaStream_t stream[2] = {nullptr, nullptr};
    cudaEvent_t in_free[2] = {nullptr, nullptr}, done[2] = {nullptr, nullptr};

    bool reserve(size_t in_bytes, size_t out_bytes);
    void release();  // the device must be current
};

// Runs `rows` rows through the device in pieces of `rows_per_piece`: rows of `in_row` bytes are copied from `in`
// into a pinned slot by parallel_copy, moved to the device, handed to `launch(d_in, d_out, first_row, nrows, stream)`,
// and the `out_row`-byte results come back the same way.  While the device works on piece p the host copies piece
// p+1 in and piece p-1 out.  Returns the first CUDA error.
using StageLaunch = std::function<cudaError_t(const void *d_in, void *d_out, int64_t first_row, int64_t nrows, cudaStream_t stream)>;
cudaError_t run_staged(StageRing &ring, const char *in, size_t in_row, char *out, size_t out_row, int64_t rows,
                       int64_t rows_per_piece, const StageLaunch &launch);

}  // namespace gguf
