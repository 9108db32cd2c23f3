/* hip/hip_runtime.h -- compatibility shim: maps the handful of HIP runtime names that the reference's launcher
 * headers (gpu_ops.h, qmatvec.h, deltanet.h) and their callers use onto the CUDA runtime, so those headers and
 * qwen_model.cpp's call sites compile unchanged against this library.
 *
 * Covered: the error type and the codes the launchers return (src/gpu_ops.cpp:68-70), the stream type, the
 * error-string call used by QwenModel::check (src/qwen_model.cpp:703-706) and the one sync per forward pass
 * (src/qwen_model.cpp:708). Anything else of HIP is outside the layer-op path. */
#ifndef B200_HIP_RUNTIME_SHIM_H
#define B200_HIP_RUNTIME_SHIM_H

#include <cuda_runtime_api.h>

typedef cudaError_t hipError_t;
typedef cudaStream_t hipStream_t;
typedef cudaEvent_t hipEvent_t;

#define hipSuccess cudaSuccess
#define hipErrorInvalidValue cudaErrorInvalidValue
#define hipErrorInvalidDeviceFunction cudaErrorInvalidDeviceFunction
#define hipErrorOutOfMemory cudaErrorMemoryAllocation

#define hipGetErrorString cudaGetErrorString
#define hipGetLastError cudaGetLastError
#define hipDeviceSynchronize cudaDeviceSynchronize
#define hipStreamSynchronize cudaStreamSynchronize
#define hipMalloc cudaMalloc
#define hipFree cudaFree
#define hipMemcpy cudaMemcpy
#define hipMemcpyAsync cudaMemcpyAsync
#define hipMemcpyHostToDevice cudaMemcpyHostToDevice
#define hipMemcpyDeviceToHost cudaMemcpyDeviceToHost
#define hipMemcpyDeviceToDevice cudaMemcpyDeviceToDevice
#define hipMemsetAsync cudaMemsetAsync

#endif
