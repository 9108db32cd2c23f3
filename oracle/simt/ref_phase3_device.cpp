// The reference's FP16 component kernels (src/layernorm.hip "rmsnorm", src/rope_embedding.hip "rope_rotate_half"),
// compiled unchanged as host C++ against the SIMT emulation of this folder. Test infrastructure only.
#include <hip/hip_runtime.h>
#include <hip/hip_fp16.h>

#include "layernorm.hip"
#include "rope_embedding.hip"

SIMT_KERNEL(rmsnorm) SIMT_KERNEL(rope_rotate_half)
