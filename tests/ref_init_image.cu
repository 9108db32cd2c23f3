// Test scaffolding, not part of the library: the module image tests/test_gpu_reference_launchers.py hands to the
// reference's own gpu_ops.cpp. That file's gpu_ops_init refuses a module that lacks any of the 23 kernel names it looks
// up (src/gpu_ops.cpp:26-48), twenty of which belong to model families outside this library's path. The image is
// therefore the library's named kernels (add_rmsnorm, add_rmsnorm_rows, swiglu, ...) plus EMPTY kernels under the
// other twenty names, present only so that the reference's init succeeds; the test launches none of them.
#include "named_kernels.cu"

#define PLACEHOLDER(name) extern "C" __global__ void name() {}
PLACEHOLDER(moe_router) PLACEHOLDER(moe_combine) PLACEHOLDER(moe_group) PLACEHOLDER(hc_norm) PLACEHOLDER(hc_lowrank)
PLACEHOLDER(hc_mix) PLACEHOLDER(ple_gate) PLACEHOLDER(ple_conv) PLACEHOLDER(mtp_concat) PLACEHOLDER(add_normed)
PLACEHOLDER(gemma_attn_post) PLACEHOLDER(gemma_ffn_post) PLACEHOLDER(mamba_conv) PLACEHOLDER(mamba_conv_state)
PLACEHOLDER(mamba_scan) PLACEHOLDER(mamba_gnorm) PLACEHOLDER(moe_router_sigmoid) PLACEHOLDER(relu2) PLACEHOLDER(geglu)
PLACEHOLDER(softcap)
