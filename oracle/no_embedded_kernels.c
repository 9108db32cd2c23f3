/* no_embedded_kernels.c -- the symbols the reference's kernel_loader.cpp expects from its kernels_embed.S
 * (src/kernel_loader.cpp:10-15), all empty: with nothing embedded the loader takes a module from
 * $INFERENCE_KERNEL_DIR/<name> or the working directory (src/kernel_loader.cpp:31-39), which is where the tests put
 * this library's module images. Test infrastructure: linked only into oracle/_ref/libref_gpu_ops.so. */
const char inference_co_matvec_q[1] = {0}, inference_co_matvec_q_end[1] = {0};
const char inference_co_gpu_ops[1] = {0}, inference_co_gpu_ops_end[1] = {0};
const char inference_co_deltanet[1] = {0}, inference_co_deltanet_end[1] = {0};
const char inference_co_attention[1] = {0}, inference_co_attention_end[1] = {0};
