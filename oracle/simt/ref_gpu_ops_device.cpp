// ref_gpu_ops_device.cpp -- compiles the REFERENCE'S OWN device code, src/gpu_ops.hip (with src/q8_device.h), unchanged
// and where it lies (the Makefile passes its directory with -I), for the host SIMT emulation of this folder, and makes
// its kernels launchable by the names the reference's launchers look up (src/gpu_ops.cpp:26-48). Test infrastructure.
#include <hip/hip_runtime.h>

#include "gpu_ops.hip"

SIMT_KERNEL(add_rmsnorm) SIMT_KERNEL(add_rmsnorm_rows) SIMT_KERNEL(swiglu) SIMT_KERNEL(moe_router)
SIMT_KERNEL(moe_combine) SIMT_KERNEL(moe_group) SIMT_KERNEL(hc_norm) SIMT_KERNEL(hc_lowrank) SIMT_KERNEL(hc_mix)
SIMT_KERNEL(ple_gate) SIMT_KERNEL(ple_conv) SIMT_KERNEL(mtp_concat) SIMT_KERNEL(add_normed)
SIMT_KERNEL(gemma_attn_post) SIMT_KERNEL(gemma_ffn_post) SIMT_KERNEL(mamba_conv) SIMT_KERNEL(mamba_conv_state)
SIMT_KERNEL(mamba_scan) SIMT_KERNEL(mamba_gnorm) SIMT_KERNEL(moe_router_sigmoid) SIMT_KERNEL(relu2) SIMT_KERNEL(geglu)
SIMT_KERNEL(softcap)
