// internal.h -- what the translation units of libb200_layer_ops.so share besides the public header: the library's
// initialisation state and its launch counter (both live in layer_ops.cu).

#ifndef B200_INTERNAL_H
#define B200_INTERNAL_H

#include <cuda_runtime_api.h>

namespace b200 {

// gpu_ops_init has succeeded and gpu_ops_free has not been called since: every launcher returns
// cudaErrorInvalidDeviceFunction while this is false (src/gpu_ops.cpp:68,81)
bool lib_ready();

// Counts one kernel launch (b200_launch_count) and returns the launch status (cudaGetLastError)
cudaError_t launched();

}  // namespace b200

#endif  // B200_INTERNAL_H
