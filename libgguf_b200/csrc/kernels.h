// Internal launch interface between the C-ABI layer and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gguf {

// Dequantize `nelems` elements (a whole number of blocks) of `type` from device memory.
// out_dtype: 0 fp32, 1 fp16, 2 bf16.  Asynchronous on `stream`.
cudaError_t launch_dequantize(int type, const void *src, void *dst, int64_t nelems, int out_dtype, cudaStream_t stream);

// True if launch_quantize has a kernel for this type.
bool quantize_supported(int type);
// fp16 (src_dtype 1) / bf16 (2) -> fp32, n values
// acc[c] += sum over rows (in row order) of rows[r][c]^2
cudaError_t launch_sumsq_columns(const float *rows, int64_t nrows, int64_t n, float *acc, cudaStream_t stream);
cudaError_t launch_widen(int src_dtype, const void *src, float *dst, int64_t n, cudaStream_t stream);

// Quantizers that stage their input with bulk asynchronous copies (TQ1_0, TQ2_0, Q1_0) count, on the device, the
// waits for a copy that ran out; a CTA that gave up leaves its part of the output unwritten.  Host paths that
// synchronise the stream read the counter of the current device before and after and fail the call when it moved.
bool uses_bulk_staging(int type);
cudaError_t read_staging_timeouts(unsigned long long *count);
// limit < 0 restores the default; 0 makes every consumer give up at once (test hook, current device)
cudaError_t set_staging_wait_limit(int limit);

// Launch accounting (exposed through libgguf_cuda_kernel_launch_count).
void count_launch();

#ifdef __CUDACC__
// Programmatic dependent launch.  A kernel started with launch_overlapped() may become resident while
// the previous kernel of the stream is still draining; it must call grid_dependency_wait() before its
// first access to global memory (the call returns once the previous kernel has completed and its
// writes are visible, or at once when there is nothing to wait for), so stream order is kept.
// grid_dependents_may_launch() tells the scheduler that the kernel after this one may start to be
// placed on SMs as they become free.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... KArgs, class... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(block);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}
#endif
uint64_t launch_count();

}  // namespace gguf
