// The reference's attention device code (src/attention.hip, with src/q8_device.h) compiled unchanged as host C++
// against the SIMT emulation of this folder, for the attn_prep kernels: q / k norm + RoPE, the Hadamard rotation and
// the FP16 / Q8_0 / Q4_0 cache rows. Test infrastructure only.
#include <hip/hip_runtime.h>
#include <hip/hip_fp16.h>

// The file's two clang vector typedefs (16 x _Float16, 8 x float) are both 32 bytes: gcc's spelling of the same.
// They serve the matrix-instruction kernels only, which compile here and are not run.
#define ext_vector_type(N) vector_size(32)

#include "attention.hip"

SIMT_KERNEL(attn_prep_64) SIMT_KERNEL(attn_prep_128) SIMT_KERNEL(attn_prep_256) SIMT_KERNEL(attn_prep_512)
