// named_attn.cu -- "attn_prep_64", "attn_prep_128", "attn_prep_256", "attn_prep_512": the first kernel of the
// reference's attention (src/attention.hip:266-300, entry points :969-977), looked up by name in its attention
// module (src/attention.cpp:55-58) and launched with grid (n_q + n_kv, T), block D (src/attention.cpp:155-158). Same
// names, argument list and launch geometry, for a caller that keeps the reference's module-launch code. Per token z
// (position pos0 + z):
//   blocks b <  n_q : q head b  -> bias, RMSNorm * q_norm, RoPE -> q_out (rotated by the Hadamard block when ATTN_KV_ROT)
//   blocks b >= n_q : kv head g -> K: bias, RMSNorm * k_norm, RoPE; V: bias, optional plain RMSNorm; both written
//                     to their cache rows as fp16, or quantised to Q8_0 / Q4_0 (after the rotation when ATTN_KV_ROT)
// A compatibility kernel in the reference's one-value-per-thread shape; the arithmetic is this library's: sums of
// squares in double and 1/rms as the CPU reference forms it (src/qwen_ops.cpp:8-11), the angle pos * base^(-2i/n_rot)
// as a double product, cos / sin in double rounded once, every product and sum of the rotation rounded on its own
// (src/qwen_ops.cpp:15-24), the quantisers of kv_store.cuh. Built into attention.fatbin.

#include "common.cuh"
#include "kv_store.cuh"

using namespace b200;

namespace {

#define ATTN_KV_ROT 4

// Sum over the D threads of the CTA; every call ends with a barrier, so the buffer can be reused at once
template <int D>
__device__ __forceinline__ double head_sum(double v, double* part) {
    v = group_sum(v, 32);
    if (D == 32) return v;
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int k = 0; k < D / 32; ++k) tot += part[k];
    __syncthreads();
    return tot;
}

// RMSNorm (gamma w or none; skipped unless norm) then RoPE of one head held one value per thread. NeoX pairs
// (i, i + n_rot / 2), or (2 i, 2 i + 1) with rope_norm; pair i < rot_pairs turns by pos * base^(-2 i / n_rot) / ff[i].
template <int D>
__device__ __forceinline__ float norm_rope_value(float x, const float* w, int n_rot, int rot_pairs, int pos, float freq_base,
                                                 float eps, bool norm, int rope_norm, const float* ff, float* xs,
                                                 double* part) {
    const int d = threadIdx.x;
    if (norm) {  // uniform
        const float inv = inv_rms(head_sum<D>((double)x * (double)x, part), 1.0 / (double)D, eps);
        x = __fmul_rn(__fmul_rn(x, inv), w ? w[d] : 1.0f);
    }
    xs[d] = x;
    __syncthreads();
    const int half = n_rot / 2;
    const int i = rope_norm ? d / 2 : (d < half ? d : d - half);
    if (d < n_rot && i < rot_pairs) {
        double theta = (double)pos * pow((double)freq_base, -2.0 * (double)i / (double)n_rot);
        if (ff) theta /= (double)ff[i];
        double ds, dc;
        sincos(theta, &ds, &dc);
        const float sn = (float)ds, cs = (float)dc;
        const int i0 = rope_norm ? 2 * i : i, i1 = rope_norm ? 2 * i + 1 : i + half;
        const float x0 = xs[i0], x1 = xs[i1];
        x = d == i0 ? __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)) : __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
    }
    __syncthreads();
    return x;
}

// The reference's Hadamard rotation of the head's D values in blocks of N, one value per thread: butterflies
// s = 1 .. N / 2 in order through shared memory (src/attention.hip:251-263)
template <int D>
__device__ __forceinline__ float rot_value(float x, int N, float* xs) {
    const int d = threadIdx.x;
    for (int s = 1; s < N; s <<= 1) {
        xs[d] = x;
        __syncthreads();
        const float y = xs[d ^ s];
        x = (d & s) ? __fsub_rn(y, x) : __fadd_rn(x, y);
        __syncthreads();
    }
    return __fmul_rn(x, __fdiv_rn(1.0f, __fsqrt_rn((float)N)));
}

__device__ __forceinline__ int rot_block_of(int D) {
    int r = 64;
    while (D % (2 * r) == 0) r *= 2;
    return r;
}

// Value x as element e of a quantised cache row; the 32 lanes of a warp hold one block (src/attention.hip:159-178)
__device__ __forceinline__ void store_quantised(__half* row_h, int e, float x, int kq, int kv_stride) {
    uint8_t* row = reinterpret_cast<uint8_t*>(row_h);
    const int lane = e & 31;
    float amax = fabsf(x);
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (kq == 1) {
        const int d_row = kv_stride * 32 / 17;
        const float d = __fdiv_rn(amax, 127.0f);
        reinterpret_cast<int8_t*>(row)[e] = (int8_t)__float2int_rn(d != 0.0f ? __fmul_rn(x, __fdiv_rn(1.0f, d)) : 0.0f);
        if (lane == 0) reinterpret_cast<__half*>(row + d_row)[e / 32] = __float2half_rn(d);
    } else {
        const int d_row = kv_stride * 32 / 9;
        float m = fabsf(x) == amax ? x : -INFINITY;
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        const float d = __fdiv_rn(m, -8.0f);
        const int n = min(15, (int)(d != 0.0f ? __fadd_rn(__fmul_rn(x, __fdiv_rn(1.0f, d)), 8.5f) : 8.0f));
        const int hi = __shfl_down_sync(0xffffffffu, n, 4);
        if ((e & 4) == 0) row[(e >> 3) * 4 + (e & 3)] = (uint8_t)(n | (hi << 4));
        if (lane == 0) reinterpret_cast<__half*>(row + d_row / 2)[e / 32] = __float2half_rn(d);
    }
}

template <int D>
__device__ __forceinline__ void attn_prep(const float* qfull, const float* k, const float* v, const float* q_norm,
                                          const float* k_norm, float* q_out, __half* K, __half* V, int kv_stride,
                                          int kv_shift, long long kv_bstride, int n_q, int n_kv, int n_rot, int pos0,
                                          float freq_base, float eps, int gated, int rot_pairs, int v_norm, int qk_norm,
                                          int kv_quant, const float* bq, const float* bk, const float* bv,
                                          int rope_norm, const float* ff) {
    __shared__ float xs[D];
    __shared__ double part[D / 32];
    const int b = blockIdx.x, d = threadIdx.x, z = blockIdx.y, pos = pos0 + z;
    const int qs = gated ? 2 * D : D;
    const bool rot = (kv_quant & ATTN_KV_ROT) != 0;
    if (b < n_q) {
        const size_t in = ((size_t)z * n_q + b) * qs + d;
        const float x = bq ? __fadd_rn(qfull[in], bq[(size_t)b * qs + d]) : qfull[in];
        float y = norm_rope_value<D>(x, q_norm, n_rot, rot_pairs, pos, freq_base, eps, qk_norm != 0, rope_norm, ff, xs, part);
        if (rot) y = rot_value<D>(y, rot_block_of(D), xs);
        q_out[((size_t)z * n_q + b) * D + d] = y;
        return;
    }
    const int g = b - n_q, e = g * D + d;
    const size_t in = (size_t)z * n_kv * D + e;
    float kx = bk ? __fadd_rn(k[in], bk[e]) : k[in];
    kx = norm_rope_value<D>(kx, k_norm, n_rot, rot_pairs, pos, freq_base, eps, qk_norm != 0, rope_norm, ff, xs, part);
    if (rot) kx = rot_value<D>(kx, rot_block_of(D), xs);
    float vx = bv ? __fadd_rn(v[in], bv[e]) : v[in];
    if (v_norm) vx = norm_rope_value<D>(vx, nullptr, 0, 0, pos, freq_base, eps, true, 0, nullptr, xs, part);
    if (rot) vx = rot_value<D>(vx, 64, xs);
    __half* k_row = K + kv_row(pos, kv_stride, kv_shift, kv_bstride);
    __half* v_row = V + kv_row(pos, kv_stride, kv_shift, kv_bstride);
    if (kv_quant & 3) {
        store_quantised(k_row, e, kx, kv_quant & 3, kv_stride);
        store_quantised(v_row, e, vx, kv_quant & 3, kv_stride);
    } else {
        k_row[e] = __float2half_rn(kx);
        v_row[e] = __float2half_rn(vx);
    }
}

}  // namespace

#define ATTN_PREP_KERNEL(D)                                                                                             \
    extern "C" __global__ void __launch_bounds__(D)                                                                    \
    attn_prep_##D(const float* qfull, const float* k, const float* v, const float* q_norm, const float* k_norm,         \
                  float* q_out, __half* K, __half* V, int kv_stride, int kv_shift, long long kv_bstride, int n_q,       \
                  int n_kv, int n_rot, int pos0, float freq_base, float eps, int gated, int rot_pairs, int v_norm,      \
                  int qk_norm, int kv_quant, const float* bq, const float* bk, const float* bv, int rope_norm,          \
                  const float* ff) {                                                                                    \
        attn_prep<D>(qfull, k, v, q_norm, k_norm, q_out, K, V, kv_stride, kv_shift, kv_bstride, n_q, n_kv, n_rot, pos0, \
                     freq_base, eps, gated, rot_pairs, v_norm, qk_norm, kv_quant, bq, bk, bv, rope_norm, ff);           \
    }

ATTN_PREP_KERNEL(64)
ATTN_PREP_KERNEL(128)
ATTN_PREP_KERNEL(256)
ATTN_PREP_KERNEL(512)
