/* oracle_ops.h -- CPU restatement of the reference's per-token layer ops. TEST INFRASTRUCTURE ONLY.
 *
 * This is the checker for the CUDA kernels, never the product: only the test suite, the smoke check and
 * the benchmark's cpu_baseline / reference arm may link or load it. Every function names the reference
 * file:line whose arithmetic it restates. Built with -O2 -ffp-contract=off so that no host ever fuses a
 * multiply-add the reference evaluates as two roundings.
 *
 * Parity pin: the restatement is compared bit for bit with the reference's own qwen_ops.cpp /
 * quant_types.cpp compiled from source (oracle/_ref) and with golden vectors generated from that build
 * (tests/golden). The two FP16 component-test references (layernorm_verify / rope_verify) exist in the
 * reference only inside GPU test programs, so those are pinned procedurally: same LCG, same shapes,
 * same pass rule.
 */
#ifndef ORACLE_OPS_H
#define ORACLE_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids (src/quant_types.h:19-41) of the row formats the embedding gather decodes */
#define ORC_F32 0
#define ORC_F16 1
#define ORC_Q4_0 2
#define ORC_Q4_1 3
#define ORC_Q5_0 6
#define ORC_Q5_1 7
#define ORC_Q8_0 8
#define ORC_Q4_K 12
#define ORC_Q5_K 13
#define ORC_Q6_K 14
#define ORC_BF16 30

/* ---- scalar conversions */
float    orc_fp16_to_fp32(uint16_t h);   /* src/quant_types.cpp:16-40 */
uint16_t orc_fp32_to_fp16(float f);      /* IEEE round-to-nearest-even, what __half(float) does on the host */
float    orc_bf16_to_fp32(uint16_t h);   /* src/quant_types.cpp:42-47 */
uint16_t orc_fp32_to_bf16(float f);      /* src/q8_device.h:37-41 (RNE on the bit pattern) */

/* ---- RMSNorm (src/qwen_ops.cpp:8-13) and the fused residual add (src/gpu_ops.hip:36,50-53) */
void orc_rmsnorm(const float* x, const float* w, float* y, int n, float eps);
/* T rows of n: x_out = x_in + add (only when add != NULL; x_out then written), y = rmsnorm(x_out) * w */
void orc_add_rmsnorm(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, int T,
                     float eps);
/* bf16 storage, fp32 arithmetic: the sum is rounded to bf16, stored, and the norm consumes the stored value */
void orc_add_rmsnorm_bf16(const uint16_t* x_in, const uint16_t* add, uint16_t* x_out, const float* w, uint16_t* y,
                          int n, int T, float eps);

/* ---- SwiGLU (src/qwen_ops.h:47, tests/forward_verify.cpp:365) */
float orc_silu(float x);
void orc_swiglu(const float* g, const float* u, float* out, int64_t n);
void orc_swiglu_bf16(const uint16_t* g, const uint16_t* u, uint16_t* out, int64_t n);
/* rows whose gate / up halves sit at strides (the experts' fused [gate | up] rows; src/gpu_ops.hip:659-671 shape) */
void orc_swiglu_strided(const float* gate, const float* up, float* out, int rows, int h, int64_t gate_stride,
                        int64_t up_stride);

/* ---- NeoX RoPE (src/qwen_ops.cpp:15-24); rot_pairs / freq factors as src/attention.hip:223-231 and
 *      tests/forward_verify.cpp:846-852 (pairs >= rot_pairs stay; theta / ff[i]) */
void orc_rope_neox(float* v, int n_rot, int pos, float freq_base);
void orc_rope_neox_ex(float* v, int n_rot, int rot_pairs, int pos, float freq_base, const float* ff);

/* ---- per-head q/k RMSNorm -> RoPE (tests/forward_verify.cpp:835-853 qk_ref; src/attention.hip:266-283 for the
 *      gated head stride). qfull [T][n_q * (gated ? 2 D : D)], k [T][n_kv * D]; q_out [T][n_q * D], k_out [T][n_kv * D].
 *      positions NULL: row t is at pos0 + t. q_norm / k_norm NULL: no gamma. do_norm 0: RoPE only. */
void orc_qk_norm_rope(const float* qfull, const float* k, const float* q_norm, const float* k_norm, float* q_out,
                      float* k_out, int n_q, int n_kv, int D, int n_rot, int rot_pairs, const int* positions,
                      int pos0, int T, float freq_base, float eps, int gated, const float* ff, int do_norm);
void orc_qk_norm_rope_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                           uint16_t* q_out, uint16_t* k_out, int n_q, int n_kv, int D, int n_rot, int rot_pairs,
                           const int* positions, int pos0, int T, float freq_base, float eps, int gated,
                           const float* ff, int do_norm);

/* ---- GGUF block decoders (src/quant_types.cpp:78-91,181-189,635-646) and the gather loop
 *      (src/qwen_model.cpp:980-986; embd_scale as :1405-1409). Return 0, or -1 for a bad type / size / token id. */
size_t orc_row_size(int type, int64_t ne0);
int orc_to_float(int type, const void* src, float* dst, int64_t n);
int orc_embed_rows(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens, float* out, int E,
                   int T, float scale);
int orc_embed_rows_bf16(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens,
                        uint16_t* out, int E, int T, float scale);

/* ---- the two FP16 component-test references
 *      tests/layernorm_verify.cpp:70-76 (sequential fp32 sum, 1/sqrtf, one rounding) */
void orc_rmsnorm_f16(const uint16_t* x, const uint16_t* gamma, uint16_t* y, int n_tokens, int n_embd, float eps);
/*      tests/rope_verify.cpp:73-81 (tables in double, stored fp32) and :84-93 (rotate-half on the tables) */
void orc_rope_tables(const int* positions, int n_rows, int dim, float theta, float* ctab, float* stab);
void orc_rope_rotate_half_f16(const uint16_t* x, const float* ctab, const float* stab, uint16_t* y, int n_rows,
                              int half_dim);
/*      the tests' LCG (tests/layernorm_verify.cpp:29-33): advances *state, returns a value in [lo, hi) */
float orc_lcg(uint32_t* state, float lo, float hi);

/* ---- activation side outputs of the producers (src/q8_device.h:54-104): per 256-value block b of the flattened
 *      vector. Any output pointer may be NULL. K must be a multiple of 256 (of 32 when only q0 / d0 / s0 are wanted). */
void orc_quantize_q8(const float* x, int64_t K, int8_t* q0, float* d0, int32_t* s0, int8_t* qK, float* dK,
                     int32_t* bsK, uint16_t* xh, int xh_bf16);

#ifdef __cplusplus
}
#endif

#endif /* ORACLE_OPS_H */
