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

/* The module-launch and pinned-host calls of the reference's component test programs
 * (tests/layernorm_verify.cpp:78-98, tests/rope_verify.cpp:95-116) and of its launcher sources (src/gpu_ops.cpp,
 * src/kernel_loader.cpp), onto the CUDA driver's module API and the
 * runtime's host registration, so that those programs compile unchanged and load this library's module images in
 * place of their .co files. Off unless B200_HIP_SHIM_MODULE_API is defined: it needs cuda.h and -lcuda. */
#ifdef B200_HIP_SHIM_MODULE_API
#include <cuda.h>

typedef CUmodule hipModule_t;
typedef CUfunction hipFunction_t;
#define hipHostRegisterDefault cudaHostRegisterDefault
#define hipHostRegister cudaHostRegister
#define hipHostUnregister cudaHostUnregister
#define hipHostGetDevicePointer cudaHostGetDevicePointer

static inline hipError_t b200_hip_from_cu(CUresult r) { return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorUnknown; }
static inline hipError_t hipInit(unsigned flags) {
    const CUresult r = cuInit(flags);
    if (r != CUDA_SUCCESS) return cudaErrorUnknown;
    return cudaFree(0);   /* the driver calls below need the runtime's primary context current on this thread */
}
static inline hipError_t hipModuleLoadData(hipModule_t* mod, const void* image) {
    if (cudaFree(0) != cudaSuccess) return cudaErrorUnknown;
    return b200_hip_from_cu(cuModuleLoadData(mod, image));
}
static inline hipError_t hipModuleLoad(hipModule_t* mod, const char* path) {
    if (cudaFree(0) != cudaSuccess) return cudaErrorUnknown;   /* (makes the primary context current) */
    return b200_hip_from_cu(cuModuleLoad(mod, path));
}
static inline hipError_t hipModuleGetFunction(hipFunction_t* fn, hipModule_t mod, const char* name) {
    return b200_hip_from_cu(cuModuleGetFunction(fn, mod, name));
}
static inline hipError_t hipModuleLaunchKernel(hipFunction_t fn, unsigned gx, unsigned gy, unsigned gz, unsigned bx,
                                               unsigned by, unsigned bz, unsigned shared_bytes, hipStream_t stream,
                                               void** params, void** extra) {
    return b200_hip_from_cu(cuLaunchKernel(fn, gx, gy, gz, bx, by, bz, shared_bytes, stream, params, extra));
}
static inline hipError_t hipModuleUnload(hipModule_t mod) { return b200_hip_from_cu(cuModuleUnload(mod)); }
#endif

#endif
