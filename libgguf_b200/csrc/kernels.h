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

// Launch accounting (exposed through libgguf_cuda_kernel_launch_count).
void count_launch();
uint64_t launch_count();

}  // namespace gguf
