#include "device_state.h"
#include "kernels.h"
namespace gguf {
cudaError_t launch_quantize_iq1(int, const float *, const float *, void *, int64_t, int64_t, const DeviceState *, cudaStream_t) { return cudaErrorNotSupported; }
}
