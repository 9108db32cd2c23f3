/* b200_layer_ops.h -- C ABI of libb200_layer_ops.so: the fused per-token layer kernels (RMSNorm with optional
 * residual add, per-head q/k norm + NeoX RoPE, SwiGLU, Q8_0 / Q4_0 embedding gather) for NVIDIA B200 (sm_100a).
 *
 * Part 1 re-declares, with identical names, argument order and meaning, the launchers of the reference engine's
 * gpu_ops module (src/gpu_ops.h:16-125; the two its Qwen forward pass calls first, then the MoE, Gemma-4,
 * hyper-connection / PLE / MTP and Mamba-2 ones): a build of the reference's qwen_model.cpp that includes its own
 * gpu_ops.h through the hip/ shim headers next to this file links against this library unchanged. hipError_t is
 * cudaError_t and hipStream_t is cudaStream_t there, as here.
 * Part 2 declares what the reference does elsewhere than in a launcher of its own (bf16 rows, the q/k norm + RoPE and
 * the KV-cache row writes it runs inside attn_prep, the embedding decode it runs in a host loop, the FP16 component
 * kernels it launches by name) and is additive. Part 3: the same operations on host buffers, streamed through one or
 * several GPUs. Part 4: reading a GGUF file's tensor table and uploading a tensor.
 *
 * Conventions, all from the reference (src/gpu_ops.h:1-2, src/gpu_ops.cpp:66-86): every pointer is device memory
 * owned by the caller unless a parameter says "host"; launches are asynchronous on `stream` and never synchronise;
 * no launcher allocates; errors come back as the return value (cudaErrorInvalidDeviceFunction before gpu_ops_init,
 * cudaErrorInvalidValue for arguments the contract forbids, otherwise the launch status), nothing is thrown or
 * printed.
 */
#ifndef B200_LAYER_OPS_H
#define B200_LAYER_OPS_H

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------ Part 1 */

/* Activation side outputs a producer kernel can write in the same launch (layout of the reference's
 * struct qmatvec_q8, src/qmatvec.h:70-83; skipped when the reference's own header was included first). */
#ifndef QMATVEC_H
typedef struct qmatvec_q8 {
    int8_t* q0;    /* Q8_0 values [K] */
    float* d0;     /* Q8_0 scales [K / 32], fp16-rounded */
    int8_t* qK;    /* Q8_K values [K] */
    float* dK;     /* Q8_K scales [K / 256] */
    int32_t* bsK;  /* Q8_K sums of every 16 values [K / 16] */
    int32_t* s0;   /* per 32 values: fp16(d * sum of the block's q) as float bits */
    int max_k;
    uint16_t* xh;  /* optional: the values rounded to bf16 (xh_bf16) or fp16 [K] */
    int xh_bf16;
} qmatvec_q8;
#endif

/* src/gpu_ops.h:16-18, src/gpu_ops.cpp:19-64. The kernels are linked into the library (the counterpart of the
 * reference's embedded code objects), so co_path is accepted and ignored; returns 0 when the current device can run
 * them, -1 otherwise; idempotent. gpu_ops_free forgets the initialisation. */
int gpu_ops_init(const char* co_path);
void gpu_ops_free(void);

/* src/gpu_ops.h:20-25. T rows of n fp32 values: x_out = x_in + add, y = RMSNorm(x_out) * w (w NULL: no gamma).
 * add NULL: x_out is not written and may be anything, y = RMSNorm(x_in) * w, and y may be x_in. x_out must not be
 * x_in when add is set. q8 non-NULL: the rows of y are also written into it as one flattened [T * n] vector
 * (n % 256 == 0 and T * n <= q8->max_k, else cudaErrorInvalidValue). */
cudaError_t gpu_add_rmsnorm(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, int T,
                            float eps, const qmatvec_q8* q8, cudaStream_t stream);

/* src/gpu_ops.h:27-29. out = SiLU(g) * u over n fp32 values; q8 non-NULL: also quantised into it
 * (n % 32 == 0 and n <= q8->max_k, else cudaErrorInvalidValue). */
cudaError_t gpu_swiglu(const float* g, const float* u, float* out, int n, const qmatvec_q8* q8, cudaStream_t stream);

/* src/gpu_ops.h:66-77, src/gpu_ops.cpp:115-122. Groups the T * n_used (token, slot) entries of ids [T][n_used] by
 * expert for expert-tiled consumers: tok_rows[i] = token, pair_rows[i] = token * n_used + slot of the i-th entry in
 * expert order (tok_rows / pair_rows: T * n_used ints); each expert's run cut into tiles of up to `tile` entries,
 * tile_e / tile_start / tile_n (gpu_moe_max_tiles entries each), *n_tiles of them. n_expert <= 1024. Unlike the
 * reference, the order inside an expert's run is fixed too (ascending pair index). Batches of more than 8192 entries
 * are grouped by three launches over the whole device and need n_segments * n_expert ints of work memory: this entry
 * point takes it from four slots inside the library (4 MiB each, part of the library image on every GPU that loads
 * it), used in turn: at most four such groupings may be in flight on a device at once, a fifth overlapping call would
 * share counters with the first; a CUDA-graph capture bakes the slot of its capture-time call into the graph, so
 * replays may meet other users of that slot. Callers that cannot keep to that pass their own work memory
 * (gpu_moe_group_scratch below). */
#ifndef GPU_OPS_H
static inline int gpu_moe_max_tiles(int T, int n_used, int n_expert, int tile) {
    const int n = T * n_used, bound = n_expert + n / tile;
    return n < bound ? n : bound;
}
#endif
cudaError_t gpu_moe_group(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows,
                          int* n_tiles, int* tile_e, int* tile_start, int* tile_n, cudaStream_t stream);

/* The sibling chains of the reference's Gemma-4 layers, same signatures and argument rules (src/gpu_ops.h:48-68,
 * src/gpu_ops.cpp:186-234; kernels src/gpu_ops.hip:521-606,659-677). Rows [T][n] fp32, n % 256 == 0, n <= 4096.
 *   gpu_add_normed:       out = (base + RMSNorm(a) * w) * (*scale, or 1 if NULL); out may be base, not a.
 *   gpu_gemma_attn_post:  x_out = x + RMSNorm(a) * w_a; y1 = RMSNorm(x_out) * w1 (side outputs into q8 if set);
 *                         y2 = RMSNorm(x_out) * w2 if w2. x_out is neither x nor a.
 *   gpu_geglu:            out [rows][h] = GELU_tanh(g) * u, g / u row r at gate + r * gate_stride / up + r * up_stride
 *                         (strides >= h; the experts' fused [gate | up] rows: up = gate + h, strides 2 h).
 *   gpu_softcap:          x = cap * tanh(x / cap) in place, cap > 0.
 *   gpu_moe_combine[_scaled]: out [T][n] = sum_j wts[t][j] * down[t][j] (+ sg[t] * shared[t]; + shared[t] if sg is
 *                         NULL; wts NULL: weight 1), down [T][n_used][n], in slot order; _scaled: each expert's
 *                         output times exp_scale[ids[t][j]] first (src/gpu_ops.h:40-46). Any n.
 *   gpu_gemma_ffn_post:   c = the combine above (no shared expert); h = RMSNorm(mlp) * w1 + RMSNorm(c) * w2;
 *                         x_out = (x + RMSNorm(h) * w_post) * (*scale, or 1); y = RMSNorm(x_out) * w_next (side
 *                         outputs into q8 if set). x_out is not x.
 *   gpu_moe_router:       per token, p = softmax(logits [T][n_expert]); ids / wts [T][n_used] = the n_used largest p in
 *                         descending order (ties to the lower index) and p / max(their sum, 2^-14); with w_shexp,
 *                         sg[t] = sigmoid(x[t] . w_shexp) (x [T][n]); ids_stride (0: n_used) > n_used: ids rows of
 *                         ids_stride entries, entry n_used set to -1. n_expert <= 1024, n_used <= 64
 *                         (src/gpu_ops.h:30-37).
 *   gpu_moe_router_sigmoid: p = sigmoid(logits); the n_used largest p + bias; weights p, divided by max(sum, 2^-14)
 *                         if norm, times scale (src/gpu_ops.h:119-123).
 *   gpu_relu2:            out [rows][h] = max(x, 0)^2, row r of x at in + r * stride (side outputs into q8 if set).
 * cudaErrorInvalidValue for the reference's refusals and for NULL or not 16-byte aligned row pointers. */
cudaError_t gpu_add_normed(const float* base, const float* a, const float* w, const float* scale, float* out, int n, int T,
                           float eps, cudaStream_t stream);
cudaError_t gpu_gemma_attn_post(const float* x, const float* a, const float* w_a, float* x_out, const float* w1, float* y1,
                                const qmatvec_q8* q8, const float* w2, float* y2, int n, int T, float eps,
                                cudaStream_t stream);
cudaError_t gpu_gemma_ffn_post(const float* x, const float* mlp, const float* down, const float* wts, const int* ids,
                               const float* exp_scale, int n_used, const float* w1, const float* w2, const float* w_post,
                               const float* scale, float* x_out, const float* w_next, float* y, const qmatvec_q8* q8, int n,
                               int T, float eps, cudaStream_t stream);
cudaError_t gpu_moe_router(const float* logits, const float* x, const float* w_shexp, int* ids, float* wts, float* sg,
                           int n_expert, int n_used, int n, int T, cudaStream_t stream, int ids_stride);
cudaError_t gpu_moe_router_sigmoid(const float* logits, const float* bias, int* ids, float* wts, int n_expert, int n_used,
                                   int norm, float scale, int T, cudaStream_t stream);
cudaError_t gpu_relu2(const float* in, float* out, int rows, int h, int stride, const qmatvec_q8* q8, cudaStream_t stream);
cudaError_t gpu_moe_combine(const float* down, const float* wts, const float* shared, const float* sg, float* out,
                            int n_used, int n, int T, cudaStream_t stream);
cudaError_t gpu_moe_combine_scaled(const float* down, const float* wts, const float* shared, const float* sg,
                                   const int* ids, const float* exp_scale, float* out, int n_used, int n, int T,
                                   cudaStream_t stream);
cudaError_t gpu_geglu(const float* gate, const float* up, float* out, int rows, int h, int gate_stride, int up_stride,
                      const qmatvec_q8* q8, cudaStream_t stream);
cudaError_t gpu_softcap(float* x, int n, float cap, cudaStream_t stream);

/* The remaining row-parallel launchers of the reference's gpu_ops module, same signatures and argument rules
 * (src/gpu_ops.h:78-105,117; src/gpu_ops.cpp:124-184,260-270; kernels src/gpu_ops.hip:322-476,763-792). The residual of
 * a hyper-connection model is hc streams of n values per token, rows r = t * hc + c.
 *   gpu_hc_norm:     with cur [T][n]: res_out[r] = res_in[r] + cur[t] * 2 * sigmoid(inject[r] / hc) first (res_out may be
 *                    res_in); y[r] = RMSNorm(that) * w[c * n ..] (side outputs into q8 over the flattened
 *                    [T * hc * n]). n % 256 == 0, n <= 4096.
 *   gpu_hc_lowrank:  out [T][np] = SiLU(lo [T][n] / hc), zero-padded to rows of np >= n.
 *   gpu_hc_mix:      out[t] = mean over the streams c of xn[r] * sigmoid(gate[r]).
 *   gpu_ple_gate:    key, res, gated, normed [T][hc][n]; value [T][n]; gammas [hc * n]: per stream
 *                    s = (RMSNorm(key) * wk) . (RMSNorm(res) * wq) / sqrt(n), g = sigmoid(sgn(s) * sqrt(max(|s|, 1e-6))),
 *                    gated = value * g, normed = RMSNorm(gated) * wc.
 *   gpu_mtp_concat:  out [T][hc][2 n] = [e[t] | h[t][c]].
 *   gpu_mamba_gnorm: out [T][d_inner] = RMSNorm(y * SiLU(z)) * w per group of d_inner / n_group values (a multiple of
 *                    256, at most 1024), z at the start of zx's rows (stride ld). */
/* The kernels of the same module that look back over earlier tokens (src/gpu_ops.h:96-116; src/gpu_ops.cpp:168-176,
 * 236-258; kernels src/gpu_ops.hip:476-512,679-760), same signatures:
 *   gpu_mamba_conv: out [T][conv_dim] = SiLU(causal conv1d of zx's xBC columns (at x_off, row stride ld) + bias),
 *                   2 <= d_conv <= 8 taps, w [conv_dim][d_conv]; conv_state [conv_dim][d_conv - 1] holds the inputs
 *                   before the batch and is advanced.
 *   gpu_mamba_scan: the selective scan, state [n_head][64][128] (d_inner = 64 n_head), B / C of group h / (n_head /
 *                   n_group) from xbc [T][d_inner + 256 n_group], dt from zx at dt_off: y [T][d_inner].
 *   gpu_ple_conv:   res += gated + SiLU(dilated causal depthwise conv of normed), m channels, K fp16 taps w [m][K];
 *                   state [(K - 1) dil][m] is advanced; state_mid (or NULL): p[j] receives the state after token j. */
#ifndef DELTANET_H   /* (src/deltanet.h:19-21; include the reference's header first when both are used) */
typedef struct deltanet_mid_states { float* p[3]; } deltanet_mid_states;
#endif
cudaError_t gpu_mamba_conv(const float* zx, long long ld, int x_off, float* conv_state, const float* w, const float* bias,
                           float* out, int conv_dim, int d_conv, int T, cudaStream_t stream);
cudaError_t gpu_mamba_scan(float* state, const float* xbc, const float* zx, long long ld, int dt_off, const float* dt_b,
                           const float* A, const float* D, float* y, int n_head, int d_inner, int n_group, int T,
                           cudaStream_t stream);
cudaError_t gpu_ple_conv(const float* normed, const float* gated, float* res, float* state, const void* w, int m, int T,
                         int K, int dil, const deltanet_mid_states* state_mid, cudaStream_t stream);
cudaError_t gpu_hc_norm(const float* res_in, float* res_out, const float* cur, const float* inject, const float* w, float* y,
                        int n, int hc, int T, float eps, const qmatvec_q8* q8, cudaStream_t stream);
cudaError_t gpu_hc_lowrank(const float* lo, float* out, int n, int np, int T, int hc, const qmatvec_q8* q8,
                           cudaStream_t stream);
cudaError_t gpu_hc_mix(const float* xn, const float* gate, float* out, int n, int hc, int T, const qmatvec_q8* q8,
                       cudaStream_t stream);
cudaError_t gpu_ple_gate(const float* key, const float* value, const float* res, const float* wk, const float* wq,
                         const float* wc, float* gated, float* normed, int n, int hc, int T, float eps,
                         cudaStream_t stream);
cudaError_t gpu_mtp_concat(const float* e, const float* h, float* out, int n, int hc, int T, cudaStream_t stream);
cudaError_t gpu_mamba_gnorm(const float* y, const float* zx, long long ld, const float* w, float* out, int d_inner,
                            int n_group, int T, float eps, const qmatvec_q8* q8, cudaStream_t stream);

/* ------------------------------------------------------------------------------------------------ Part 2 */

/* bf16 storage (uint16_t bit patterns), fp32 arithmetic, one round-to-nearest-even per stored value (the rule of
 * src/q8_device.h:39-40). The norm is taken of x_out as stored. Gammas stay fp32 as in the reference's models.
 * T and n are 64-bit / int as the tensors of a long prefill need. */
cudaError_t gpu_add_rmsnorm_bf16(const uint16_t* x_in, const uint16_t* add, uint16_t* x_out, const float* w,
                                 uint16_t* y, int n, long long T, float eps, cudaStream_t stream);
cudaError_t gpu_swiglu_bf16(const uint16_t* g, const uint16_t* u, uint16_t* out, long long n, cudaStream_t stream);
/* gpu_add_rmsnorm / gpu_swiglu without the int limits on T and n (no q8) */
cudaError_t gpu_add_rmsnorm_f32(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n,
                                long long T, float eps, cudaStream_t stream);
cudaError_t gpu_swiglu_f32(const float* g, const float* u, float* out, long long n, cudaStream_t stream);

/* SwiGLU over rows whose gate and up halves sit at strides (in values), e.g. the experts' fused [gate | up] rows:
 * out [rows][h] = SiLU(gate[r * gate_stride + i]) * up[r * up_stride + i] (argument order of the reference's
 * gpu_geglu, src/gpu_ops.h:66-67, with SiLU as the activation). */
cudaError_t gpu_swiglu_rows(const float* gate, const float* up, float* out, long long rows, int h,
                            long long gate_stride, long long up_stride, cudaStream_t stream);
cudaError_t gpu_swiglu_rows_bf16(const uint16_t* gate, const uint16_t* up, uint16_t* out, long long rows, int h,
                                 long long gate_stride, long long up_stride, cudaStream_t stream);

/* Per-head q/k RMSNorm followed by NeoX RoPE: the norm_rope step of the reference's attn_prep kernels
 * (src/attention.hip:212-236, 266-283; arguments named as in attention_forward_opts, src/attention.h:90-94) without
 * the KV-cache write. For each of T tokens: the n_q heads of qfull (head stride 2 * head_dim when gated, else
 * head_dim) go to q_out [T][n_q * head_dim], the n_kv heads of k to k_out [T][n_kv * head_dim]. Each head is
 * RMS-normalised with q_norm / k_norm (NULL: no gamma; qk_norm 0: no normalisation at all), then pairs
 * (i, i + n_rot / 2), i < rot_pairs, are rotated by pos * freq_base^(-2 i / n_rot) (/ freq_factors[i] if given);
 * rot_pairs <= 0 means n_rot / 2; n_rot 0 means no rotation. Token t is at positions[t], or at pos0 + t when
 * positions is NULL. Angles are formed and evaluated in double precision. In place (q_out == qfull without gated,
 * k_out == k) is allowed. n_kv may be 0 with k, k_out NULL (and likewise n_q). */
cudaError_t gpu_qk_norm_rope(const float* qfull, const float* k, const float* q_norm, const float* k_norm,
                             float* q_out, float* k_out, int n_q, int n_kv, int head_dim, int n_rot, int rot_pairs,
                             const int* positions, int pos0, long long T, float freq_base, float eps, int gated,
                             int qk_norm, const float* freq_factors, cudaStream_t stream);
cudaError_t gpu_qk_norm_rope_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                  uint16_t* q_out, uint16_t* k_out, int n_q, int n_kv, int head_dim, int n_rot,
                                  int rot_pairs, const int* positions, int pos0, long long T, float freq_base,
                                  float eps, int gated, int qk_norm, const float* freq_factors, cudaStream_t stream);

/* The same with the cos / sin of the angles taken from tables, so that a forward pass evaluates them once and every
 * layer's call only streams rows (the reference's FP16 component kernel takes host-built tables the same way,
 * src/rope_embedding.hip:18-37, tests/rope_verify.cpp:73-81).
 * gpu_rope_table fills cos_tab / sin_tab [T][n_rot / 2] fp32 (device memory, caller-owned): row t = token t at
 * positions[t] (or pos0 + t), entry i = cos / sin of the double-precision angle pos * freq_base^(-2 i / n_rot)
 * (/ freq_factors[i]), rounded once; pairs at or beyond rot_pairs hold (1, 0). n_rot 0: nothing to do.
 * gpu_qk_norm_rope_tab[_bf16] is gpu_qk_norm_rope with positions, base, factors and rot_pairs replaced by the tables
 * (NULL allowed when n_rot is 0): the same results as gpu_qk_norm_rope given the same angles. */
cudaError_t gpu_rope_table(const int* positions, int pos0, long long T, int n_rot, int rot_pairs, float freq_base,
                           const float* freq_factors, float* cos_tab, float* sin_tab, cudaStream_t stream);
cudaError_t gpu_qk_norm_rope_tab(const float* qfull, const float* k, const float* q_norm, const float* k_norm,
                                 float* q_out, float* k_out, int n_q, int n_kv, int head_dim, int n_rot,
                                 const float* cos_tab, const float* sin_tab, long long T, float eps, int gated,
                                 int qk_norm, cudaStream_t stream);
cudaError_t gpu_qk_norm_rope_tab_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                      uint16_t* q_out, uint16_t* k_out, int n_q, int n_kv, int head_dim, int n_rot,
                                      const float* cos_tab, const float* sin_tab, long long T, float eps, int gated,
                                      int qk_norm, cudaStream_t stream);

/* gpu_qk_norm_rope with the K write of the reference's attn_prep folded in (src/attention.hip:286-299, FP16 cache):
 * the K heads go, rounded to fp16, straight to row pos_t of k_cache (the layer's K row 0; row addressing as
 * gpu_kv_store_f16 below) instead of a k_out tensor, so K makes no extra round trip; q as in gpu_qk_norm_rope. fp32
 * rows: the same bits as gpu_qk_norm_rope followed by gpu_kv_store_f16; bf16 rows: K is rounded once, from fp32 to fp16
 * (not to bf16 on the way). kv_stride >= n_kv * head_dim. V rows: gpu_kv_store_f16. */
cudaError_t gpu_qk_norm_rope_kv(const float* qfull, const float* k, const float* q_norm, const float* k_norm, float* q_out,
                                uint16_t* k_cache, int kv_stride, int kv_shift, long long kv_bstride, int n_q, int n_kv,
                                int head_dim, int n_rot, int rot_pairs, const int* positions, int pos0, long long T,
                                float freq_base, float eps, int gated, int qk_norm, const float* freq_factors,
                                cudaStream_t stream);
cudaError_t gpu_qk_norm_rope_kv_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                     uint16_t* q_out, uint16_t* k_cache, int kv_stride, int kv_shift, long long kv_bstride,
                                     int n_q, int n_kv, int head_dim, int n_rot, int rot_pairs, const int* positions,
                                     int pos0, long long T, float freq_base, float eps, int gated, int qk_norm,
                                     const float* freq_factors, cudaStream_t stream);

/* The two combined: cos / sin from the tables of gpu_rope_table (row t = token t), K into the FP16 cache at row
 * positions[t] (or pos0 + t). The same bits as gpu_qk_norm_rope_kv given the same angles. */
cudaError_t gpu_qk_norm_rope_tab_kv(const float* qfull, const float* k, const float* q_norm, const float* k_norm,
                                    float* q_out, uint16_t* k_cache, int kv_stride, int kv_shift, long long kv_bstride,
                                    int n_q, int n_kv, int head_dim, int n_rot, const float* cos_tab, const float* sin_tab,
                                    const int* positions, int pos0, long long T, float eps, int gated, int qk_norm,
                                    cudaStream_t stream);
cudaError_t gpu_qk_norm_rope_tab_kv_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                         uint16_t* q_out, uint16_t* k_cache, int kv_stride, int kv_shift,
                                         long long kv_bstride, int n_q, int n_kv, int head_dim, int n_rot,
                                         const float* cos_tab, const float* sin_tab, const int* positions, int pos0,
                                         long long T, float eps, int gated, int qk_norm, cudaStream_t stream);

/* The whole first stage of the reference's attention for an FP16 cache (attn_prep, src/attention.hip:266-300, without
 * biases, V norm and interleaved pairs): gpu_qk_norm_rope_kv for q and K, then the V rows (v [T][n_kv * head_dim]) into
 * V; two launches on `stream`. K and V are the layer's row 0 of the two halves of the cache. */
cudaError_t gpu_attn_prep_f16(const float* qfull, const float* k, const float* v, const float* q_norm, const float* k_norm,
                              float* q_out, uint16_t* K, uint16_t* V, int kv_stride, int kv_shift, long long kv_bstride,
                              int n_q, int n_kv, int head_dim, int n_rot, int rot_pairs, const int* positions, int pos0,
                              long long T, float freq_base, float eps, int gated, int qk_norm, const float* freq_factors,
                              cudaStream_t stream);
cudaError_t gpu_attn_prep_f16_bf16(const uint16_t* qfull, const uint16_t* k, const uint16_t* v, const float* q_norm,
                                   const float* k_norm, uint16_t* q_out, uint16_t* K, uint16_t* V, int kv_stride,
                                   int kv_shift, long long kv_bstride, int n_q, int n_kv, int head_dim, int n_rot,
                                   int rot_pairs, const int* positions, int pos0, long long T, float freq_base, float eps,
                                   int gated, int qk_norm, const float* freq_factors, cudaStream_t stream);

/* The K / V write of the reference's attn_prep kernels for an unquantised (FP16) cache (src/attention.hip:279-300):
 * row t of src [T][n_vals] (n_vals = n_kv * head_dim; K after gpu_qk_norm_rope, V as projected) is rounded to fp16 and
 * stored at cache + kv_row(pos_t), kv_row(p) = (p >> kv_shift) * kv_bstride + (p & ((1 << kv_shift) - 1)) * kv_stride
 * in fp16 units (src/attention.hip:38-42; a contiguous cache has kv_shift = 30), pos_t = positions[t] or pos0 + t.
 * cache is the layer's K (or V) row 0 (uint16_t = fp16 bits). 0 <= kv_shift <= 30, kv_stride >= n_vals. */
cudaError_t gpu_kv_store_f16(const float* src, uint16_t* cache, int n_vals, const int* positions, int pos0, long long T,
                             int kv_stride, int kv_shift, long long kv_bstride, cudaStream_t stream);
cudaError_t gpu_kv_store_f16_bf16(const uint16_t* src, uint16_t* cache, int n_vals, const int* positions, int pos0,
                                  long long T, int kv_stride, int kv_shift, long long kv_bstride, cudaStream_t stream);

/* The same write for a quantised cache (kv_quant 1: Q8_0, 2: Q4_0; kvq_store, src/attention.hip:159-178, row layout
 * :44-50): a row holds d_row values and then one fp16 scale per 32; kv_stride (still in fp16 units) = d_row * 17 / 32
 * (Q8_0) or d_row * 9 / 32 (Q4_0). Q8_0: d = amax / 127, q = rint(x / d). Q4_0: d = m / -8 (m the value of largest
 * magnitude), nibble = min(15, (int)(x / d + 8.5)), byte 4 j + k holding values 8 j + k (low) and 8 j + k + 4 (high).
 * n_vals % 32 == 0 and n_vals <= d_row (the reference's caches have d_row % 256 == 0, src/kv_cache.cpp:123). */
cudaError_t gpu_kv_store_q(const float* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                           int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, cudaStream_t stream);
cudaError_t gpu_kv_store_q_bf16(const uint16_t* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                                int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, cudaStream_t stream);

/* gpu_moe_group with the caller's work memory, for a host that keeps more than four long groupings in flight on one
 * device at a time (different streams) or wants none of the library's: scratch holds at least
 * gpu_moe_group_scratch_ints(T, n_used, n_expert) ints (0 for batches of up to 8192 entries; then scratch may be
 * NULL). Same results as gpu_moe_group. */
size_t gpu_moe_group_scratch_ints(int T, int n_used, int n_expert);
cudaError_t gpu_moe_group_scratch(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows,
                                  int* n_tiles, int* tile_e, int* tile_start, int* tile_n, int* scratch,
                                  size_t scratch_ints, cudaStream_t stream);

/* The rotation the reference applies for a quantised cache (ATTN_KV_ROT; hadamard_rot, src/attention.hip:238-263,
 * 285-293): an orthonormal Walsh-Hadamard transform in blocks of `block` values (64, 128, 256 or 512), its own inverse.
 * q and K rows are rotated in blocks of hadamard_k(head_dim) (64 doubled while it divides head_dim), V in blocks of
 * 64. gpu_hadamard_rot: rows of D values (D % block == 0), out may be x. gpu_kv_store_q_rot: gpu_kv_store_q with
 * the values rotated in blocks of rot_block (n_vals % rot_block == 0; 0: none) before they are quantised. */
cudaError_t gpu_hadamard_rot(const float* x, float* out, long long rows, int D, int block, cudaStream_t stream);
cudaError_t gpu_hadamard_rot_bf16(const uint16_t* x, uint16_t* out, long long rows, int D, int block, cudaStream_t stream);
cudaError_t gpu_kv_store_q_rot(const float* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                               int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, int rot_block,
                               cudaStream_t stream);
cudaError_t gpu_kv_store_q_rot_bf16(const uint16_t* src, void* cache, int n_vals, const int* positions, int pos0,
                                    long long T, int kv_stride, int kv_shift, long long kv_bstride, int kv_quant,
                                    int rot_block, cudaStream_t stream);

/* Token-embedding gather + dequantisation: out row t = decode(table row tokens[t]) * scale, the loop of
 * src/qwen_model.cpp:980-986 (scale: embd_scale of :1409; pass 1 for none). type: a ggml id of src/quant_types.h:19-41:
 * 8 (Q8_0) and 2 (Q4_0), the formats the path is measured on, and the other formats a token_embd.weight comes in:
 * 0 (F32), 1 (F16), 30 (BF16), 3 (Q4_1), 6 (Q5_0), 7 (Q5_1), 12 (Q4_K), 13 (Q5_K), 14 (Q6_K), each decoded as the
 * reference's qt_to_float decodes it (src/quant_types.cpp:58-345); row_bytes as qt_row_size(type, E) or larger (a row
 * stride); E % 32 == 0 (E % 256 == 0 for the K formats).
 * tokens are device memory. bad_row: device int the caller sets to INT_MAX beforehand; an id outside [0, vocab)
 * zero-fills its output row and lowers *bad_row to that row's index (the reference returns an error for such an id
 * before decoding anything; read the flag after the stream is synchronised). Bit-exact. */
cudaError_t gpu_embed_rows(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens, float* out,
                           int E, long long T, float scale, int* bad_row, cudaStream_t stream);
cudaError_t gpu_embed_rows_bf16(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens,
                                uint16_t* out, int E, long long T, float scale, int* bad_row, cudaStream_t stream);
/* The same with the ids in host memory, as the reference's forward() receives them: the ids are range-checked on the
 * host first (cudaErrorInvalidValue and nothing launched if one is out of range, as src/qwen_model.cpp:981), then
 * copied to tokens_dev (device scratch for T ids, caller-owned) on `stream`, and the gather is launched.
 * tokens_host must stay valid until that copy has run (pinned memory makes it asynchronous). */
cudaError_t gpu_embed_rows_host_ids(int type, const void* table, size_t row_bytes, int vocab,
                                    const int32_t* tokens_host, int32_t* tokens_dev, float* out, int E, long long T,
                                    float scale, int* bad_row, cudaStream_t stream);

/* No counterpart in the reference. gpu_embed_rows_host_ids for a caller that cannot supply device scratch (an engine
 * that handed out all of HBM at start-up, a serving loop where cudaMalloc is off limits): the device copy of the ids
 * and the bad-id flag live in an array built into the library, so the call allocates nothing and takes no scratch
 * arguments. Limits: T <= 262144 ids per call (cudaErrorInvalidValue beyond that; the array costs every GPU that
 * loads the library 1 MiB for the life of the process); all calls on a device share the array, so calls whose GPU work
 * may overlap race.
 * Ids are range-checked on the host first: an id outside [0, vocab) returns cudaErrorInvalidValue and queues nothing.
 * tokens_host must stay valid until its copy has run on `stream`. fp32 output, same bits as gpu_embed_rows. Tables of
 * type 8 (Q8_0) and 2 (Q4_0) only: any other type is cudaErrorInvalidValue (use gpu_embed_rows_host_ids for those).
 * cudaErrorInvalidDeviceFunction before gpu_ops_init, like every launcher. */
cudaError_t gpu_embed_rows_static_scratch(int type, const void* table, size_t row_bytes, int vocab,
                                          const int32_t* tokens_host, float* out, int E, long long T, float scale,
                                          cudaStream_t stream);

/* FP16 component kernels of the reference (src/layernorm.hip:15-45, src/rope_embedding.hip:18-37), which its tests
 * launch by name with one 32-thread block per row; these launchers run better-shaped kernels with the same math.
 * gpu_rmsnorm_f16: y = x * rsqrt(mean(x^2) + eps) * gamma (gamma fp16, NULL: none), fp32 accumulation, one rounding.
 * gpu_rope_rotate_half_f16: y[r][i] = x[r][i] c - x[r][i+H] s, y[r][i+H] = x[r][i+H] c + x[r][i] s with fp32 tables
 * ctab / stab [n_rows][half_dim]; y may be x. */
cudaError_t gpu_rmsnorm_f16(const uint16_t* x, const uint16_t* gamma, uint16_t* y, int n_tokens, int n_embd, float eps,
                            cudaStream_t stream);
cudaError_t gpu_rope_rotate_half_f16(const uint16_t* x, const float* ctab, const float* stab, uint16_t* y, int n_rows,
                                     int half_dim, cudaStream_t stream);

/* ------------------------------------------------------------------------------------------------ Part 3 */

/* Host-buffer entry points: the same operations for a caller whose rows live in HOST memory, as the reference's CPU
 * functions take them (qwen_rmsnorm / qwen_rope_neox / qwen_silu, src/qwen_ops.h:17-48; the gather loop,
 * src/qwen_model.cpp:980-986). A context owns, on the device that was current when it was created, `n_slots` staging
 * slots of `slot_bytes` each and one stream per slot. A call cuts the rows into chunks that fit a slot and runs
 * chunk after chunk through copy-in -> kernel -> copy-out, slot after slot, so that the copies of one chunk overlap
 * the kernel and the copies of its neighbours. Calls are synchronous: they return when the outputs are in host
 * memory. Page-locked host buffers make the copies asynchronous (pageable ones work, without overlap). One call at a
 * time per context. Row pointers are host memory; the embedding table is device memory (a weight, uploaded once).
 * Errors: cudaErrorInvalidValue for bad arguments or a row too large for a slot, else the first CUDA error met. */
typedef struct b200_host_ctx b200_host_ctx;
/* How a call cuts T rows into chunks for a ring of n_slots slots of slot_rows rows each (small chunks first and last,
 * so that little time goes to the copy in that nothing overlaps and to the last copy out; large ones in between).
 * Writes up to max_sizes chunk sizes and returns their count. Host logic only: no device is touched. */
int b200_host_chunk_plan(long long T, long long slot_rows, int n_slots, long long* sizes, int max_sizes);
b200_host_ctx* b200_host_ctx_create(size_t slot_bytes, int n_slots);   /* NULL on failure */
void b200_host_ctx_destroy(b200_host_ctx* ctx);

/* elem: 4 = fp32 rows, 2 = bf16 rows (bit patterns), as the device launchers of parts 1 and 2 */
cudaError_t b200_host_add_rmsnorm(b200_host_ctx* ctx, int elem, const void* x_in, const void* add, void* x_out,
                                  const float* w, void* y, int n, long long T, float eps);
cudaError_t b200_host_swiglu(b200_host_ctx* ctx, int elem, const void* g, const void* u, void* out, long long rows,
                             int width);
cudaError_t b200_host_qk_norm_rope(b200_host_ctx* ctx, int elem, const void* qfull, const void* k, const float* q_norm,
                                   const float* k_norm, void* q_out, void* k_out, int n_q, int n_kv, int head_dim,
                                   int n_rot, int rot_pairs, const int* positions, int pos0, long long T,
                                   float freq_base, float eps, int gated, int qk_norm, const float* freq_factors);
/* table_dev: device memory. tokens: host. An out-of-range id returns cudaErrorInvalidValue before anything runs. */
cudaError_t b200_host_embed_rows(b200_host_ctx* ctx, int elem, int type, const void* table_dev, size_t row_bytes,
                                 int vocab, const int32_t* tokens, void* out, int E, long long T, float scale);

/* The layer's whole op sequence in ONE call, in the order a layer of the reference's forward pass issues it around its
 * matmuls (src/qwen_model.cpp:980-990 gather + first norm; attn_prep's q/k norm + RoPE; :946-948 residual + ffn norm;
 * :951 SwiGLU; :955-957 residual + the next layer's norm). Every true input comes from host memory and every result
 * goes back to it, but the residual stream x, which the reference keeps in place between these ops (s.x / s.x_alt),
 * stays on the device between the kernels of a chunk instead of crossing the bus twice per op:
 *   x = embed(tokens) * embd_scale;            xn_attn = RMSNorm(x) * w_attn_norm;
 *   q_out, k_out = qk_norm_rope(qfull, k);     x' = x + attn_proj;  xn_ffn = RMSNorm(x') * w_ffn_norm;
 *   act = SiLU(gate) * up;                     x_out = x' + ffn_proj;  xn_next = RMSNorm(x_out) * w_next_norm.
 * Row pointers are host memory ([T] rows each), gammas host memory, table_dev device memory. Each row gets the bits
 * the six separate calls give it. Errors as the separate calls (an out-of-range id: cudaErrorInvalidValue, nothing run). */
typedef struct b200_layer_sweep {
    int elem;                 /* 4 = fp32 rows, 2 = bf16 rows */
    long long T;
    int qtype;                /* embedding table: ggml type id, device pointer, row stride, rows */
    const void* table_dev;
    size_t row_bytes;
    int vocab;
    const int32_t* tokens;    /* [T] */
    int E;
    float embd_scale;         /* 1 for none */
    const float* w_attn_norm; /* [E] each; NULL: no gamma */
    const float* w_ffn_norm;
    const float* w_next_norm;
    float eps;
    void* xn_attn;            /* out [T][E] */
    const void* qfull;        /* in [T][n_q * (gated ? 2 : 1) * head_dim] */
    const void* k;            /* in [T][n_kv * head_dim] */
    void* q_out;              /* out [T][n_q * head_dim] */
    void* k_out;              /* out [T][n_kv * head_dim] */
    const float* q_norm;      /* [head_dim] or NULL */
    const float* k_norm;
    int n_q, n_kv, head_dim, n_rot, rot_pairs;
    const int* positions;     /* [T] or NULL: pos0 + t */
    int pos0;
    float freq_base;
    int gated, qk_norm;
    const float* freq_factors;/* [n_rot / 2] or NULL */
    const void* attn_proj;    /* in [T][E] */
    void* xn_ffn;             /* out [T][E] */
    const void* gate;         /* in [T][FF] */
    const void* up;           /* in [T][FF] */
    int FF;
    void* act;                /* out [T][FF] */
    const void* ffn_proj;     /* in [T][E] */
    void* x_out;              /* out [T][E]: the residual stream after the layer */
    void* xn_next;            /* out [T][E] */
} b200_layer_sweep;
cudaError_t b200_host_layer_sweep(b200_host_ctx* ctx, const b200_layer_sweep* args);

/* The same over several GPUs of one box from one process: rows are cut into contiguous ranges, one per device, and
 * one host thread per device runs the single-device call on its range; nothing is exchanged between devices and a
 * row gets the bits one device would give it. n_devices <= 0: all visible devices. tables_dev: one device pointer
 * per device of the group (the table replicated, in device order). */
typedef struct b200_host_group b200_host_group;
b200_host_group* b200_host_group_create(int n_devices, size_t slot_bytes, int n_slots);   /* NULL on failure */
void b200_host_group_destroy(b200_host_group* grp);
int b200_host_group_size(const b200_host_group* grp);
cudaError_t b200_host_group_add_rmsnorm(b200_host_group* grp, int elem, const void* x_in, const void* add, void* x_out,
                                        const float* w, void* y, int n, long long T, float eps);
cudaError_t b200_host_group_swiglu(b200_host_group* grp, int elem, const void* g, const void* u, void* out, long long rows,
                                   int width);
cudaError_t b200_host_group_qk_norm_rope(b200_host_group* grp, int elem, const void* qfull, const void* k,
                                         const float* q_norm, const float* k_norm, void* q_out, void* k_out, int n_q,
                                         int n_kv, int head_dim, int n_rot, int rot_pairs, const int* positions, int pos0,
                                         long long T, float freq_base, float eps, int gated, int qk_norm,
                                         const float* freq_factors);
cudaError_t b200_host_group_embed_rows(b200_host_group* grp, int elem, int type, const void* const* tables_dev,
                                       size_t row_bytes, int vocab, const int32_t* tokens, void* out, int E, long long T,
                                       float scale);
/* b200_host_layer_sweep over the group's devices: device g runs rows [T g / G, T (g + 1) / G) with its own table
 * tables_dev[g] (args->table_dev is not used); positions, or pos0 + the range's first row, follow the rows. */
cudaError_t b200_host_group_layer_sweep(b200_host_group* grp, const b200_layer_sweep* args, const void* const* tables_dev);

/* ------------------------------------------------------------------------------------------------ Part 4 */

/* From a GGUF file to a device-resident table. The reference maps the file and lets kernels read weights in place
 * from unified memory (src/gguf_mmap.h:15-17; QuantWeight::row, src/inference_internal.h:33-40); here the mapping is
 * the source of one upload. A reader of the container layout only (GGUF version 2 / 3). A split model
 * (<prefix>-00001-of-0000N.gguf, split.count in its metadata) is opened by its first file, as the reference does
 * (src/gguf_mmap.h:92-95): the tensors of all N files form one table, each file has its own mapping. Tensor byte
 * sizes are known for the row formats gpu_embed_rows decodes: F32 (0), F16 (1), Q4_0 (2), Q4_1 (3), Q5_0 (6), Q5_1 (7),
 * Q8_0 (8), Q4_K (12), Q5_K (13), Q6_K (14), BF16 (30); tensors of other types are listed with nbytes 0 and cannot be
 * uploaded. b200_gguf_open returns NULL for a missing, truncated or malformed file. */
typedef struct b200_gguf b200_gguf;
b200_gguf* b200_gguf_open(const char* path);
void b200_gguf_close(b200_gguf* g);
long long b200_gguf_n_tensors(const b200_gguf* g);
unsigned b200_gguf_version(const b200_gguf* g);
size_t b200_gguf_alignment(const b200_gguf* g);      /* general.alignment, default 32 */
size_t b200_gguf_data_offset(const b200_gguf* g);    /* file offset of the data section (of the first file) */
int b200_gguf_n_files(const b200_gguf* g);           /* 1, or the files of a split model */
int b200_gguf_tensor_file(const b200_gguf* g, int idx);   /* which of them holds tensor idx (0: the one opened), or -1 */
int b200_gguf_find_tensor(const b200_gguf* g, const char* name);   /* index, or -1 */
/* Any out pointer may be NULL. ne: 4 extents (1 beyond n_dims); row_bytes: bytes of ne[0] values (qt_row_size);
 * host_data: the tensor's bytes inside the read-only mapping (valid until b200_gguf_close). Returns 0, or -1. */
int b200_gguf_tensor_info(const b200_gguf* g, int idx, const char** name, int* type, int* n_dims, long long ne[4],
                          size_t* row_bytes, size_t* nbytes, const void** host_data);
int b200_gguf_kv_u32(const b200_gguf* g, const char* key, uint32_t* out);   /* 0, or -1 if absent / other type */
int b200_gguf_kv_f32(const b200_gguf* g, const char* key, float* out);
long long b200_gguf_kv_str(const b200_gguf* g, const char* key, char* buf, size_t cap);   /* length, or -1 */
/* Allocates device memory for tensor idx (this is a loader: it does allocate), queues the copy on `stream`, and
 * returns the device pointer; release it with b200_gguf_free_tensor. The mapping must stay open until the copy ran. */
cudaError_t b200_gguf_upload_tensor(const b200_gguf* g, int idx, void** dev_ptr, cudaStream_t stream);
void b200_gguf_free_tensor(void* dev_ptr);

/* Number of kernel launches this library has issued since it was loaded (all launchers, all threads) */
unsigned long long b200_launch_count(void);
/* "sm_100a" and the like: the architecture the kernels were compiled for */
const char* b200_build_arch(void);

#ifdef __cplusplus
}
#endif

#endif /* B200_LAYER_OPS_H */
