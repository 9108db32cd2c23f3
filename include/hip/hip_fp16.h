/* hip/hip_fp16.h -- compatibility shim: lets the reference's headers (qwen_ops.h, q8_device.h users) that
 * include <hip/hip_fp16.h> compile against the CUDA toolkit. Only the __half type and its conversions are used
 * on the layer-op path. */
#ifndef B200_HIP_FP16_SHIM_H
#define B200_HIP_FP16_SHIM_H
#include <cuda_fp16.h>
#endif
