#include "kernels.h"
namespace kaio {
bool w4a16_decode_ok(const void*, const DqProblem*, int, uint32_t, uint32_t, uint32_t) { return false; }
size_t w4a16_decode_workspace_bytes(const DeviceCtx&, uint32_t, uint32_t) { return 0; }
cudaError_t launch_w4a16_decode(const DeviceCtx&, const __half*, const DqProblem&, bool, uint32_t, uint32_t, uint32_t, void*, uint32_t*, cudaStream_t) { return cudaErrorNotSupported; }
}
