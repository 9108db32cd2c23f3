/* oracle_ops.c -- see oracle_ops.h. CPU restatement of the reference's layer ops: TEST INFRASTRUCTURE ONLY,
 * never linked into the product library. Compile with -O2 -ffp-contract=off (no -ffast-math). */

#include "oracle_ops.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- scalars */

/* src/quant_types.cpp:16-40: exact widening, subnormals renormalised, inf / nan payload kept */
float orc_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while (!(m & 0x400u)) { m <<= 1; ++shift; }
            bits = sign | (uint32_t)(127 - 15 + 1 - shift) << 23 | (m & 0x3ffu) << 13;
        }
    } else if (e == 0x1f) {
        bits = sign | 0x7f800000u | m << 13;
    } else {
        bits = sign | (e + 112u) << 23 | m << 13;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* IEEE binary32 -> binary16, round to nearest even (what the tests' __half(float) does on the host) */
uint16_t orc_fp32_to_fp16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t a = u & 0x7fffffffu;
    if (a >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u | ((a >> 13) & 0x3ffu) : 0u));
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  /* rounds to >= 65520: infinity */
    if (a < 0x33000001u) return (uint16_t)sign;                /* <= 2^-25: rounds to zero */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift = e >= -14 ? 13 : 13 + (-14 - e);                /* subnormal halves lose more bits */
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    if (e >= -14) return (uint16_t)(sign | (uint32_t)(((e + 15) << 10) + (int)(q - 0x400u)));
    return (uint16_t)(sign | q);                               /* q may carry into the first normal: same bits */
}

float orc_bf16_to_fp32(uint16_t h) {
    const uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* src/q8_device.h:39-40 */
uint16_t orc_fp32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

/* ---------------------------------------------------------------- RMSNorm */

/* src/qwen_ops.cpp:8-13: double sum of squares, inv rounded to float once, (x * inv) * w left to right */
void orc_rmsnorm(const float* x, const float* w, float* y, int n, float eps) {
    double ss = 0.0;
    for (int i = 0; i < n; ++i) ss += (double)x[i] * x[i];
    const float inv = (float)(1.0 / sqrt(ss / n + eps));
    for (int i = 0; i < n; ++i) y[i] = x[i] * inv * (w ? w[i] : 1.0f);
}

/* src/gpu_ops.hip:36,50-53: v = x_in + add in fp32, stored to x_out, and the norm is of v */
void orc_add_rmsnorm(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, int T,
                     float eps) {
    for (int t = 0; t < T; ++t) {
        const float* xi = x_in + (size_t)t * n;
        float* yo = y + (size_t)t * n;
        if (add) {
            float* xo = x_out + (size_t)t * n;
            const float* a = add + (size_t)t * n;
            for (int i = 0; i < n; ++i) xo[i] = xi[i] + a[i];
            orc_rmsnorm(xo, w, yo, n, eps);
        } else {
            orc_rmsnorm(xi, w, yo, n, eps);
        }
    }
}

void orc_add_rmsnorm_bf16(const uint16_t* x_in, const uint16_t* add, uint16_t* x_out, const float* w, uint16_t* y,
                          int n, int T, float eps) {
    for (int t = 0; t < T; ++t) {
        const uint16_t* xi = x_in + (size_t)t * n;
        uint16_t* yo = y + (size_t)t * n;
        double ss = 0.0;
        for (int i = 0; i < n; ++i) {
            float v = orc_bf16_to_fp32(xi[i]);
            if (add) {
                const uint16_t r = orc_fp32_to_bf16(v + orc_bf16_to_fp32(add[(size_t)t * n + i]));
                x_out[(size_t)t * n + i] = r;
                v = orc_bf16_to_fp32(r);
            }
            ss += (double)v * v;
        }
        const float inv = (float)(1.0 / sqrt(ss / n + eps));
        for (int i = 0; i < n; ++i) {
            const float v = orc_bf16_to_fp32(add ? x_out[(size_t)t * n + i] : xi[i]);
            yo[i] = orc_fp32_to_bf16(v * inv * (w ? w[i] : 1.0f));
        }
    }
}

/* ---------------------------------------------------------------- SwiGLU */

/* src/qwen_ops.h:47 */
float orc_silu(float x) { return x / (1.0f + expf(-x)); }

/* tests/forward_verify.cpp:365: silu(g) * u */
void orc_swiglu(const float* g, const float* u, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_silu(g[i]) * u[i];
}

void orc_swiglu_bf16(const uint16_t* g, const uint16_t* u, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i)
        out[i] = orc_fp32_to_bf16(orc_silu(orc_bf16_to_fp32(g[i])) * orc_bf16_to_fp32(u[i]));
}

void orc_swiglu_strided(const float* gate, const float* up, float* out, int rows, int h, int64_t gate_stride,
                        int64_t up_stride) {
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < h; ++i)
            out[(size_t)r * h + i] = orc_silu(gate[r * gate_stride + i]) * up[r * up_stride + i];
}

/* ---------------------------------------------------------------- RoPE */

/* src/qwen_ops.cpp:15-24 */
void orc_rope_neox(float* v, int n_rot, int pos, float freq_base) {
    const int half = n_rot / 2;
    for (int i = 0; i < half; ++i) {
        const double theta = pos * pow((double)freq_base, -2.0 * i / n_rot);
        const float c = (float)cos(theta), s = (float)sin(theta);
        const float x0 = v[i], x1 = v[i + half];
        v[i] = x0 * c - x1 * s;
        v[i + half] = x0 * s + x1 * c;
    }
}

/* As above with the kernel's two extras (src/attention.hip:223-231): only pairs i < rot_pairs rotate, and
 * theta is divided by ff[i] when ff is set (tests/forward_verify.cpp:848). rot_pairs <= 0 means n_rot / 2. */
void orc_rope_neox_ex(float* v, int n_rot, int rot_pairs, int pos, float freq_base, const float* ff) {
    const int half = n_rot / 2;
    const int np = rot_pairs > 0 && rot_pairs < half ? rot_pairs : half;
    for (int i = 0; i < np; ++i) {
        double theta = pos * pow((double)freq_base, -2.0 * i / n_rot);
        if (ff) theta /= ff[i];
        const float c = (float)cos(theta), s = (float)sin(theta);
        const float x0 = v[i], x1 = v[i + half];
        v[i] = x0 * c - x1 * s;
        v[i + half] = x0 * s + x1 * c;
    }
}

/* tests/forward_verify.cpp:835-853 (qk_ref): x -> RMSNorm with the head's gamma -> NeoX RoPE at the row's position;
 * Q heads sit at stride 2 D in qfull when the projection also carries the attention gate (src/attention.hip:274). */
static void qk_head(const float* x, const float* gamma, float* out, int D, int n_rot, int rot_pairs, int pos,
                    float base, float eps, const float* ff, int do_norm) {
    if (do_norm) orc_rmsnorm(x, gamma, out, D, eps);
    else memmove(out, x, (size_t)D * sizeof(float));
    if (n_rot > 0) orc_rope_neox_ex(out, n_rot, rot_pairs, pos, base, ff);
}

void orc_qk_norm_rope(const float* qfull, const float* k, const float* q_norm, const float* k_norm, float* q_out,
                      float* k_out, int n_q, int n_kv, int D, int n_rot, int rot_pairs, const int* positions,
                      int pos0, int T, float freq_base, float eps, int gated, const float* ff, int do_norm) {
    const int qs = gated ? 2 * D : D;
    for (int t = 0; t < T; ++t) {
        const int pos = positions ? positions[t] : pos0 + t;
        for (int h = 0; h < n_q; ++h)
            qk_head(qfull + ((size_t)t * n_q + h) * qs, q_norm, q_out + ((size_t)t * n_q + h) * D, D, n_rot, rot_pairs,
                    pos, freq_base, eps, ff, do_norm);
        for (int h = 0; h < n_kv; ++h)
            qk_head(k + ((size_t)t * n_kv + h) * D, k_norm, k_out + ((size_t)t * n_kv + h) * D, D, n_rot, rot_pairs,
                    pos, freq_base, eps, ff, do_norm);
    }
}

void orc_qk_norm_rope_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                           uint16_t* q_out, uint16_t* k_out, int n_q, int n_kv, int D, int n_rot, int rot_pairs,
                           const int* positions, int pos0, int T, float freq_base, float eps, int gated,
                           const float* ff, int do_norm) {
    const int qs = gated ? 2 * D : D;
    float tmp[1024], res[1024];
    if (D > 1024) return;
    for (int t = 0; t < T; ++t) {
        const int pos = positions ? positions[t] : pos0 + t;
        for (int h = 0; h < n_q + n_kv; ++h) {
            const int isq = h < n_q, hh = isq ? h : h - n_q;
            const uint16_t* src = isq ? qfull + ((size_t)t * n_q + hh) * qs : k + ((size_t)t * n_kv + hh) * D;
            uint16_t* dst = isq ? q_out + ((size_t)t * n_q + hh) * D : k_out + ((size_t)t * n_kv + hh) * D;
            for (int i = 0; i < D; ++i) tmp[i] = orc_bf16_to_fp32(src[i]);
            qk_head(tmp, isq ? q_norm : k_norm, res, D, n_rot, rot_pairs, pos, freq_base, eps, ff, do_norm);
            for (int i = 0; i < D; ++i) dst[i] = orc_fp32_to_bf16(res[i]);
        }
    }
}

/* ---------------------------------------------------------------- GGUF blocks */

static float rd_f16(const uint8_t* p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return orc_fp16_to_fp32(h);
}

/* Values and bytes per block of the GGUF types the embedding gather decodes (src/quant_types.cpp:583-598) */
static int orc_block(int type, int* values, int* bytes) {
    switch (type) {
        case ORC_F32: *values = 1; *bytes = 4; return 1;
        case ORC_F16: *values = 1; *bytes = 2; return 1;
        case ORC_BF16: *values = 1; *bytes = 2; return 1;
        case ORC_Q4_0: *values = 32; *bytes = 18; return 1;
        case ORC_Q4_1: *values = 32; *bytes = 20; return 1;
        case ORC_Q5_0: *values = 32; *bytes = 22; return 1;
        case ORC_Q5_1: *values = 32; *bytes = 24; return 1;
        case ORC_Q8_0: *values = 32; *bytes = 34; return 1;
        case ORC_Q4_K: *values = 256; *bytes = 144; return 1;
        case ORC_Q5_K: *values = 256; *bytes = 176; return 1;
        case ORC_Q6_K: *values = 256; *bytes = 210; return 1;
        default: return 0;
    }
}

/* src/quant_types.cpp:635-639: bytes of a row of ne0 values, 0 when the type is unknown or ne0 is not whole blocks */
size_t orc_row_size(int type, int64_t ne0) {
    int v, b;
    if (!orc_block(type, &v, &b) || ne0 % v != 0) return 0;
    return (size_t)(ne0 / v) * (size_t)b;
}

/* The 6-bit scale and minimum j of a K-quant super-block's 12 packed bytes (src/quant_types.cpp:192-200) */
static void k4_scale_min(int j, const uint8_t* q, int* sc, int* mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
        *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

/* One block of `type` into y, value by value, every product, sum and difference rounded on its own (the decoders of
 * src/quant_types.cpp: plain :58-74, Q4_0 :78-91, Q4_1 :126-140, Q5_0 :142-159, Q5_1 :161-179, Q8_0 :181-189,
 * Q4_K :264-287, Q5_K :289-316, Q6_K :318-345) */
static void orc_block_to_float(int type, const uint8_t* b, float* y) {
    switch (type) {
        case ORC_F32: memcpy(y, b, 4); return;
        case ORC_F16: y[0] = rd_f16(b); return;
        case ORC_BF16: { uint16_t h; memcpy(&h, b, 2); y[0] = orc_bf16_to_fp32(h); return; }
        case ORC_Q8_0: {
            const float d = rd_f16(b);
            const int8_t* qs = (const int8_t*)(b + 2);
            for (int j = 0; j < 32; ++j) y[j] = qs[j] * d;
            return;
        }
        case ORC_Q4_0: {
            const float d = rd_f16(b);
            const uint8_t* qs = b + 2;
            for (int j = 0; j < 16; ++j) {
                y[j] = ((qs[j] & 0x0F) - 8) * d;
                y[j + 16] = ((qs[j] >> 4) - 8) * d;
            }
            return;
        }
        case ORC_Q4_1: {
            const float d = rd_f16(b), m = rd_f16(b + 2);
            const uint8_t* qs = b + 4;
            for (int j = 0; j < 16; ++j) {
                const float lo = (float)(qs[j] & 0x0F) * d, hi = (float)(qs[j] >> 4) * d;
                y[j] = lo + m;
                y[j + 16] = hi + m;
            }
            return;
        }
        case ORC_Q5_0:
        case ORC_Q5_1: {
            const int one = type == ORC_Q5_1;
            const float d = rd_f16(b), m = one ? rd_f16(b + 2) : 0.0f;
            uint32_t qh;
            memcpy(&qh, b + (one ? 4 : 2), 4);
            const uint8_t* qs = b + (one ? 8 : 6);
            for (int j = 0; j < 16; ++j) {
                const int h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
                const int x0 = (qs[j] & 0x0F) | h0, x1 = (qs[j] >> 4) | h1;
                if (one) {
                    const float lo = (float)x0 * d, hi = (float)x1 * d;
                    y[j] = lo + m;
                    y[j + 16] = hi + m;
                } else {
                    y[j] = (float)(x0 - 16) * d;
                    y[j + 16] = (float)(x1 - 16) * d;
                }
            }
            return;
        }
        case ORC_Q4_K:
        case ORC_Q5_K: {
            const int five = type == ORC_Q5_K;
            const float d = rd_f16(b), dmin = rd_f16(b + 2);
            const uint8_t* scales = b + 4;
            const uint8_t* qh = b + 16;                 /* Q5_K only */
            const uint8_t* ql = b + (five ? 48 : 16);
            for (int g = 0; g < 4; ++g) {               /* 64 values: 32 low nibbles, then 32 high nibbles */
                for (int half = 0; half < 2; ++half) {
                    int sc, mn;
                    k4_scale_min(2 * g + half, scales, &sc, &mn);
                    const float dd = d * (float)sc, mm = dmin * (float)mn;
                    for (int l = 0; l < 32; ++l) {
                        int v = half ? ql[g * 32 + l] >> 4 : ql[g * 32 + l] & 0x0F;
                        if (five && (qh[l] & ((half ? 2 : 1) << (2 * g)))) v += 16;
                        const float p = dd * (float)v;
                        y[g * 64 + half * 32 + l] = p - mm;
                    }
                }
            }
            return;
        }
        case ORC_Q6_K: {
            const float d = rd_f16(b + 208);
            const uint8_t* ql = b;
            const uint8_t* qh = b + 128;
            const int8_t* sc = (const int8_t*)(b + 192);
            for (int h = 0; h < 2; ++h)
                for (int quarter = 0; quarter < 4; ++quarter)
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t lb = ql[h * 64 + l + ((quarter & 1) ? 32 : 0)];
                        const int low = quarter < 2 ? lb & 0x0F : lb >> 4;
                        const int q = (int)(int8_t)(low | (((qh[h * 32 + l] >> (2 * quarter)) & 3) << 4)) - 32;
                        const float ds = d * (float)sc[h * 8 + l / 16 + 2 * quarter];
                        y[h * 128 + quarter * 32 + l] = ds * (float)q;
                    }
            return;
        }
        default: return;
    }
}

/* qt_to_float of src/quant_types.cpp:641-646 for the types above: n values (whole blocks) from src into y */
int orc_to_float(int type, const void* src, float* y, int64_t n) {
    int v, bb;
    if (!orc_block(type, &v, &bb) || n % v != 0) return -1;
    const uint8_t* b = (const uint8_t*)src;
    for (int64_t i = 0; i < n / v; ++i, b += bb, y += v) orc_block_to_float(type, b, y);
    return 0;
}

/* src/qwen_model.cpp:980-986: range check, decode row tokens[t] into out row t; :1409 multiplies by embd_scale
 * afterwards (a second rounding; scale 1 leaves the bits alone) */
int orc_embed_rows(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens, float* out, int E,
                   int T, float scale) {
    for (int t = 0; t < T; ++t) {
        if (tokens[t] < 0 || tokens[t] >= vocab) return -1;
        float* o = out + (size_t)t * E;
        if (orc_to_float(type, (const char*)table + (size_t)tokens[t] * row_bytes, o, E) != 0) return -1;
        if (scale != 1.0f)
            for (int i = 0; i < E; ++i) o[i] *= scale;
    }
    return 0;
}

int orc_embed_rows_bf16(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens,
                        uint16_t* out, int E, int T, float scale) {
    if (orc_row_size(type, E) == 0) return -1;
    float* row = (float*)malloc((size_t)E * sizeof(float));
    if (!row) return -1;
    for (int t = 0; t < T; ++t) {
        if (tokens[t] < 0 || tokens[t] >= vocab) { free(row); return -1; }
        orc_to_float(type, (const char*)table + (size_t)tokens[t] * row_bytes, row, E);
        for (int j = 0; j < E; ++j) {
            float v = row[j];
            if (scale != 1.0f) v *= scale;
            out[(size_t)t * E + j] = orc_fp32_to_bf16(v);
        }
    }
    free(row);
    return 0;
}

/* ---------------------------------------------------------------- FP16 component-test references */

/* tests/layernorm_verify.cpp:70-76 */
void orc_rmsnorm_f16(const uint16_t* x, const uint16_t* gamma, uint16_t* y, int n_tokens, int n_embd, float eps) {
    for (int t = 0; t < n_tokens; ++t) {
        float ssq = 0.0f;
        for (int c = 0; c < n_embd; ++c) {
            const float v = orc_fp16_to_fp32(x[(size_t)t * n_embd + c]);
            ssq += v * v;
        }
        const float inv = 1.0f / sqrtf(ssq / (float)n_embd + eps);
        for (int c = 0; c < n_embd; ++c) {
            const float g = gamma ? orc_fp16_to_fp32(gamma[c]) : 1.0f;  /* src/layernorm.hip:42 */
            y[(size_t)t * n_embd + c] = orc_fp32_to_fp16(orc_fp16_to_fp32(x[(size_t)t * n_embd + c]) * inv * g);
        }
    }
}

/* tests/rope_verify.cpp:73-81 */
void orc_rope_tables(const int* positions, int n_rows, int dim, float theta, float* ctab, float* stab) {
    const int H = dim / 2;
    const double log_theta = log((double)theta);
    for (int r = 0; r < n_rows; ++r)
        for (int i = 0; i < H; ++i) {
            const double freq = exp(-2.0 * ((double)i / (double)dim) * log_theta);
            const double angle = (double)positions[r] * freq;
            ctab[(size_t)r * H + i] = (float)cos(angle);
            stab[(size_t)r * H + i] = (float)sin(angle);
        }
}

/* tests/rope_verify.cpp:84-93 */
void orc_rope_rotate_half_f16(const uint16_t* x, const float* ctab, const float* stab, uint16_t* y, int n_rows,
                              int half_dim) {
    const int H = half_dim, dim = 2 * half_dim;
    for (int r = 0; r < n_rows; ++r)
        for (int i = 0; i < H; ++i) {
            const float lo = orc_fp16_to_fp32(x[(size_t)r * dim + i]);
            const float hi = orc_fp16_to_fp32(x[(size_t)r * dim + i + H]);
            const float c = ctab[(size_t)r * H + i], s = stab[(size_t)r * H + i];
            y[(size_t)r * dim + i] = orc_fp32_to_fp16(lo * c - hi * s);
            y[(size_t)r * dim + i + H] = orc_fp32_to_fp16(hi * c + lo * s);
        }
}

/* tests/layernorm_verify.cpp:29-33 */
float orc_lcg(uint32_t* state, float lo, float hi) {
    *state = *state * 1664525u + 1013904223u;
    return lo + ((float)(*state >> 8) / (float)(1u << 24)) * (hi - lo);
}

/* ---------------------------------------------------------------- activation side outputs */

/* src/q8_device.h:54-104, one 256-value block at a time (a trailing part of whole 32-value blocks gets the Q8_0
 * side only, as a partly active workgroup does). rintf rounds half to even, as the device's does. */
void orc_quantize_q8(const float* x, int64_t K, int8_t* q0, float* d0, int32_t* s0, int8_t* qK, float* dK,
                     int32_t* bsK, uint16_t* xh, int xh_bf16) {
    if (xh)
        for (int64_t i = 0; i < K; ++i) xh[i] = xh_bf16 ? orc_fp32_to_bf16(x[i]) : orc_fp32_to_fp16(x[i]);
    if (q0)
        for (int64_t b = 0; b < K / 32; ++b) {
            const float* v = x + b * 32;
            float am = 0.0f;
            for (int j = 0; j < 32; ++j) am = fmaxf(am, fabsf(v[j]));
            const float id = am != 0.0f ? 127.0f / am : 0.0f;
            int sum = 0;
            for (int j = 0; j < 32; ++j) {
                const int q = (int)rintf(v[j] * id);
                q0[b * 32 + j] = (int8_t)q;
                sum += q;
            }
            if (d0) d0[b] = orc_fp16_to_fp32(orc_fp32_to_fp16(am / 127.0f));
            if (s0) {
                const float s = orc_fp16_to_fp32(orc_fp32_to_fp16(am / 127.0f * (float)sum));
                memcpy(&s0[b], &s, 4);
            }
        }
    if (qK)
        for (int64_t b = 0; b < K / 256; ++b) {
            const float* v = x + b * 256;
            float fa = 0.0f, fv = 0.0f;
            for (int j = 0; j < 256; ++j)
                if (fabsf(v[j]) > fa) { fa = fabsf(v[j]); fv = v[j]; }  /* first on ties */
            float iscale = 0.0f;
            if (fa != 0.0f) iscale = -127.0f / fv;
            for (int g = 0; g < 16; ++g) {
                int s16 = 0;
                for (int j = 0; j < 16; ++j) {
                    int q = 0;
                    if (fa != 0.0f) {
                        q = (int)rintf(iscale * v[g * 16 + j]);
                        if (q > 127) q = 127;
                    }
                    qK[b * 256 + g * 16 + j] = (int8_t)q;
                    s16 += q;
                }
                if (bsK) bsK[b * 16 + g] = s16;
            }
            if (dK) dK[b] = fa != 0.0f ? 1.0f / iscale : 0.0f;
        }
}
