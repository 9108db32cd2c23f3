// norm_chains.cuh -- the sibling norm chains of the reference's Gemma-4 path, built on the same row reduction as
// rmsnorm.cuh (src/gpu_ops.hip:521-606) and its two elementwise neighbours (:659-677):
//   add_normed       out = (base + RMSNorm(a) * w) * (*scale, or 1)
//   gemma_attn_post  x_out = x + RMSNorm(a) * w_a;  y1 = RMSNorm(x_out) * w1;  y2 = RMSNorm(x_out) * w2 (if w2)
//   geglu            out = GELU_tanh(g) * u on rows whose gate / up halves sit at a stride
//   softcap          x = cap * tanh(x / cap), in place
//   moe_combine      out = sum_j wts_j * down_j (+ sg * shared), the experts' outputs back into token rows (:245-264)
//   gemma_ffn_post   the FFN epilogue: combine, two norms added, residual, scale, the next layer's norm (:608-655)
// Every product and sum is rounded on its own, in the order the reference writes them: RMSNorm(v) * w is
// (v * inv) * w, then the add, then the scale. inv = (float)(1 / sqrt(ss / n + eps)) with ss summed in double, as in
// rmsnorm.cuh, so the chains give the bits of the separate norm kernels followed by fp32 adds.
//
// Rows are [T][n] fp32 contiguous, n a multiple of 256 up to 4096 (the reference's own limits): a row is exactly
// blockDim.x * VPT 16-byte vectors, one CTA per row, each value read once and written once per output.

#ifndef B200_NORM_CHAINS_CUH
#define B200_NORM_CHAINS_CUH

#include "common.cuh"

namespace b200 {

template <int VPT>
__device__ __forceinline__ double row_sumsq(const f2 (&v)[VPT][2]) {
    double s0 = 0.0, s1 = 0.0;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        sumsq2(v[j][0], s0, s1);
        sumsq2(v[j][1], s0, s1);
    }
    return s0 + s1;
}

// a + p where p is a packed product that must keep its own rounding: a packed add straight after a packed multiply
// may be merged into one fused multiply-add by the assembler, the scalar add intrinsics never are
__device__ __forceinline__ f2 add_rounded(f2 a, f2 p) {
    float a0, a1, p0, p1;
    upk2(a, a0, a1);
    upk2(p, p0, p1);
    return pk2(__fadd_rn(a0, p0), __fadd_rn(a1, p1));
}

__device__ __forceinline__ void gamma_pair(const float* w, size_t vec, f2 (&g)[2]) {
    const ulonglong2 r = __ldg(reinterpret_cast<const ulonglong2*>(w) + vec);
    g[0] = r.x;
    g[1] = r.y;
}

template <int VPT>
__global__ void __launch_bounds__(512)
k_add_normed(const float* base, const float* a, const float* w, const float* scale, float* out, int n, long long T,
             float eps) {
    __shared__ double part[2][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const size_t row_vecs = (size_t)tpr * VPT;
    const double inv_n = 1.0 / (double)n;
    const float s = scale ? __ldg(scale) : 1.0f;
    const f2 s2 = pk2(s, s);
    int flip = 0;
    for (long long row = blockIdx.x; row < T; row += gridDim.x, flip ^= 1) {
        const size_t off = (size_t)row * row_vecs + l;
        uint4 ra[VPT], rb[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            ra[j] = ld_stream(reinterpret_cast<const uint4*>(a) + off + j * tpr);
            rb[j] = ld_stream(reinterpret_cast<const uint4*>(base) + off + j * tpr);
        }
        f2 v[VPT][2];
#pragma unroll
        for (int j = 0; j < VPT; ++j) Io2<float>::unpack(ra[j], v[j]);
        const float inv = inv_rms(cta_sum(row_sumsq<VPT>(v), part[flip]), inv_n, eps);
        const f2 inv2 = pk2(inv, inv);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g[2], b[2];
            gamma_pair(w, (size_t)l + (size_t)j * tpr, g);
            Io2<float>::unpack(rb[j], b);
#pragma unroll
            for (int k = 0; k < 2; ++k) v[j][k] = mul2(add_rounded(b[k], mul2(mul2(v[j][k], inv2), g[k])), s2);
            st_stream(reinterpret_cast<uint4*>(out) + off + j * tpr, Io2<float>::pack(v[j]));
        }
    }
}

template <int VPT>
__global__ void __launch_bounds__(512)
k_gemma_attn_post(const float* x, const float* a, const float* w_a, float* x_out, const float* w1, float* y1,
                  const float* w2, float* y2, int n, long long T, float eps) {
    __shared__ double part[2][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const size_t row_vecs = (size_t)tpr * VPT;
    const double inv_n = 1.0 / (double)n;
    for (long long row = blockIdx.x; row < T; row += gridDim.x) {
        const size_t off = (size_t)row * row_vecs + l;
        uint4 ra[VPT], rx[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            ra[j] = ld_stream(reinterpret_cast<const uint4*>(a) + off + j * tpr);
            rx[j] = ld_stream(reinterpret_cast<const uint4*>(x) + off + j * tpr);
        }
        f2 v[VPT][2];
#pragma unroll
        for (int j = 0; j < VPT; ++j) Io2<float>::unpack(ra[j], v[j]);
        const float ia = inv_rms(cta_sum(row_sumsq<VPT>(v), part[0]), inv_n, eps);
        const f2 ia2 = pk2(ia, ia);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g[2], b[2];
            gamma_pair(w_a, (size_t)l + (size_t)j * tpr, g);
            Io2<float>::unpack(rx[j], b);
#pragma unroll
            for (int k = 0; k < 2; ++k) v[j][k] = add_rounded(b[k], mul2(mul2(v[j][k], ia2), g[k]));
            st_stream(reinterpret_cast<uint4*>(x_out) + off + j * tpr, Io2<float>::pack(v[j]));
        }
        const float inv = inv_rms(cta_sum(row_sumsq<VPT>(v), part[1]), inv_n, eps);
        const f2 inv2 = pk2(inv, inv);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g[2], o[2];
            gamma_pair(w1, (size_t)l + (size_t)j * tpr, g);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                v[j][k] = mul2(v[j][k], inv2);
                o[k] = mul2(v[j][k], g[k]);
            }
            st_stream(reinterpret_cast<uint4*>(y1) + off + j * tpr, Io2<float>::pack(o));
            if (w2) {
                gamma_pair(w2, (size_t)l + (size_t)j * tpr, g);
#pragma unroll
                for (int k = 0; k < 2; ++k) o[k] = mul2(v[j][k], g[k]);
                st_stream(reinterpret_cast<uint4*>(y2) + off + j * tpr, Io2<float>::pack(o));
            }
        }
        // (the second reduction's barrier separates this row's reads of part[0] from the next row's writes)
    }
}

// ---------------------------------------------------------------- MoE combine and the FFN epilogue

// One slot's term of the experts' weighted sum for a packed pair (src/gpu_ops.hip:259-261): (d * exp_scale[e]) * w
// with per-expert scales, else w * d; the sum runs in slot order, each product and each add rounded on its own.
__device__ __forceinline__ f2 combine_term(f2 d, float w, float es, bool scaled) {
    return scaled ? mul2(mul2(d, pk2(es, es)), pk2(w, w)) : mul2(pk2(w, w), d);
}

// out [T][n] = sum_j wts[t][j] * down[t][j][:] (+ shared[t] * sg[t], or + shared[t] when sg is NULL); wts NULL: weight 1
// (src/gpu_ops.hip:245-264). down is [T][n_used][n]. One thread per 16-byte vector of out (VEC: n % 4 == 0 and
// aligned bases) or per value; up to 8 slots' loads are in flight per thread.
template <bool VEC>
__global__ void __launch_bounds__(256)
k_moe_combine(const float* down, const float* wts, const float* shared, const float* sg, float* out, int n_used, int n,
              long long T, const int* ids, const float* exp_scale) {
    const int per_row = VEC ? n / 4 : n;
    const long long total = T * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per_row;
        const int c = (int)(i - t * per_row);
        const float* w = wts ? wts + t * n_used : nullptr;
        const int* e = exp_scale ? ids + t * n_used : nullptr;
        if (VEC) {
            const uint4* d = reinterpret_cast<const uint4*>(down + (size_t)t * n_used * n) + c;
            f2 acc[2];
            for (int j0 = 0; j0 < n_used; j0 += 8) {
                uint4 r[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (j0 + u < n_used) r[u] = ld_stream(d + (size_t)(j0 + u) * per_row);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int j = j0 + u;
                    if (j < n_used) {
                        f2 v[2];
                        Io2<float>::unpack(r[u], v);
                        if (w) {
                            const float wj = __ldg(w + j), es = e ? __ldg(exp_scale + __ldg(e + j)) : 1.0f;
                            v[0] = combine_term(v[0], wj, es, e != nullptr);
                            v[1] = combine_term(v[1], wj, es, e != nullptr);
                        }
                        if (j == 0) { acc[0] = v[0]; acc[1] = v[1]; }
                        else { acc[0] = add_rounded(acc[0], v[0]); acc[1] = add_rounded(acc[1], v[1]); }
                    }
                }
            }
            if (shared) {
                f2 sv[2];
                Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(shared) + i), sv);
                if (sg && w) {
                    const float g = __ldg(sg + t);
                    sv[0] = mul2(sv[0], pk2(g, g));
                    sv[1] = mul2(sv[1], pk2(g, g));
                }
                acc[0] = add_rounded(acc[0], sv[0]);
                acc[1] = add_rounded(acc[1], sv[1]);
            }
            st_stream(reinterpret_cast<uint4*>(out) + i, Io2<float>::pack(acc));
        } else {
            const float* d = down + (size_t)t * n_used * n + c;
            float acc = 0.0f;
            for (int j = 0; j < n_used; ++j) {
                float v = d[(size_t)j * n];
                if (w) v = e ? __fmul_rn(__fmul_rn(v, exp_scale[e[j]]), w[j]) : __fmul_rn(w[j], v);
                acc = j == 0 ? v : __fadd_rn(acc, v);
            }
            if (shared) acc = __fadd_rn(acc, (sg && w) ? __fmul_rn(shared[i], sg[t]) : shared[i]);
            out[i] = acc;
        }
    }
}

// Gemma-4's norm chain after the FFN, one CTA per row (src/gpu_ops.hip:608-655):
//   c = the experts' outputs combined (as k_moe_combine: exp_scale, wts);  h = RMSNorm(mlp) * w1 + RMSNorm(c) * w2;
//   x_out = (x + RMSNorm(h) * w_post) * (*scale, or 1);  y = RMSNorm(x_out) * w_next
template <int VPT>
__global__ void __launch_bounds__(512)
k_gemma_ffn_post(const float* x, const float* mlp, const float* down, const float* wts, const int* ids,
                 const float* exp_scale, int n_used, const float* w1, const float* w2, const float* w_post,
                 const float* scale, float* x_out, const float* w_next, float* y, int n, long long T, float eps) {
    __shared__ double part[4][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const size_t row_vecs = (size_t)tpr * VPT;
    const double inv_n = 1.0 / (double)n;
    const float sc = scale ? __ldg(scale) : 1.0f;
    for (long long row = blockIdx.x; row < T; row += gridDim.x) {
        const size_t off = (size_t)row * row_vecs + l;
        f2 h[VPT][2], c[VPT][2];
        const float* wt = wts + row * n_used;
        const int* e = ids + row * n_used;
        const uint4* d = reinterpret_cast<const uint4*>(down) + (size_t)row * n_used * row_vecs + l;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            for (int u0 = 0; u0 < n_used; u0 += 4) {   // four slots' vectors in flight per row vector
                uint4 r[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (u0 + k < n_used) r[k] = ld_stream(d + (size_t)(u0 + k) * row_vecs + j * tpr);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int u = u0 + k;
                    if (u < n_used) {
                        f2 v[2];
                        Io2<float>::unpack(r[k], v);
                        const float wu = __ldg(wt + u), es = exp_scale ? __ldg(exp_scale + __ldg(e + u)) : 1.0f;
                        v[0] = combine_term(v[0], wu, es, exp_scale != nullptr);
                        v[1] = combine_term(v[1], wu, es, exp_scale != nullptr);
                        if (u == 0) { c[j][0] = v[0]; c[j][1] = v[1]; }
                        else { c[j][0] = add_rounded(c[j][0], v[0]); c[j][1] = add_rounded(c[j][1], v[1]); }
                    }
                }
            }
        }
        // (the dense MLP's row is fetched after the experts' so that its registers are not held through the combine)
#pragma unroll
        for (int j = 0; j < VPT; ++j) Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(mlp) + off + j * tpr), h[j]);
        const float im = inv_rms(cta_sum(row_sumsq<VPT>(h), part[0]), inv_n, eps);
        const float ic = inv_rms(cta_sum(row_sumsq<VPT>(c), part[1]), inv_n, eps);
        const f2 im2 = pk2(im, im), ic2 = pk2(ic, ic);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g1[2], g2[2];
            gamma_pair(w1, (size_t)l + (size_t)j * tpr, g1);
            gamma_pair(w2, (size_t)l + (size_t)j * tpr, g2);
#pragma unroll
            for (int k = 0; k < 2; ++k)
                h[j][k] = add_rounded(mul2(mul2(h[j][k], im2), g1[k]), mul2(mul2(c[j][k], ic2), g2[k]));
        }
        const float ih = inv_rms(cta_sum(row_sumsq<VPT>(h), part[2]), inv_n, eps);
        const f2 ih2 = pk2(ih, ih), sc2 = pk2(sc, sc);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g[2], b[2];
            gamma_pair(w_post, (size_t)l + (size_t)j * tpr, g);
            Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(x) + off + j * tpr), b);
#pragma unroll
            for (int k = 0; k < 2; ++k) h[j][k] = mul2(add_rounded(b[k], mul2(mul2(h[j][k], ih2), g[k])), sc2);
            st_stream(reinterpret_cast<uint4*>(x_out) + off + j * tpr, Io2<float>::pack(h[j]));
        }
        const float inv = inv_rms(cta_sum(row_sumsq<VPT>(h), part[3]), inv_n, eps);
        const f2 inv2 = pk2(inv, inv);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g[2], o[2];
            gamma_pair(w_next, (size_t)l + (size_t)j * tpr, g);
#pragma unroll
            for (int k = 0; k < 2; ++k) o[k] = mul2(mul2(h[j][k], inv2), g[k]);
            st_stream(reinterpret_cast<uint4*>(y) + off + j * tpr, Io2<float>::pack(o));
        }
        // (four buffers: a row's reductions are separated from the next row's by the barriers in between)
    }
}

// GELU, tanh form, times u: 0.5 x (1 + tanh(0.79788456 x (1 + 0.044715 x x))) * u, products left to right
// (src/gpu_ops.hip:665-667)
__device__ __forceinline__ float gelu_tanh_mul(float x, float u) {
    const float inner = __fmul_rn(__fmul_rn(0.7978845608028654f, x),
                                  __fadd_rn(1.0f, __fmul_rn(__fmul_rn(0.044715f, x), x)));
    const float g = __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner)));
    return __fmul_rn(g, u);
}

// VEC: h, both strides and all bases multiples of four values
template <bool VEC>
__global__ void __launch_bounds__(256)
k_geglu(const float* gate, const float* up, float* out, long long rows, int h, long long gate_stride, long long up_stride) {
    const int per_row = VEC ? h / 4 : h;
    const long long total = rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / per_row;
        const int c = (int)(i - r * per_row);
        if (VEC) {
            float g[4], u[4];
            Io<float>::unpack(ld_stream(gate + r * gate_stride + c * 4), g);
            Io<float>::unpack(ld_stream(up + r * up_stride + c * 4), u);
#pragma unroll
            for (int e = 0; e < 4; ++e) g[e] = gelu_tanh_mul(g[e], u[e]);
            st_stream(out + r * (long long)h + c * 4, Io<float>::pack(g));
        } else {
            out[i] = gelu_tanh_mul(gate[r * gate_stride + c], up[r * up_stride + c]);
        }
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
k_softcap(float* x, long long n, float cap) {
    const long long total = VEC ? n / 4 : n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        if (VEC) {
            float v[4];
            Io<float>::unpack(ld_stream(x + i * 4), v);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = __fmul_rn(cap, tanhf(__fdiv_rn(v[e], cap)));
            st_stream(x + i * 4, Io<float>::pack(v));
        } else {
            x[i] = __fmul_rn(cap, tanhf(__fdiv_rn(x[i], cap)));
        }
    }
    if (VEC && blockIdx.x == 0 && threadIdx.x < (int)(n - total * 4)) {
        const long long i = total * 4 + threadIdx.x;
        x[i] = __fmul_rn(cap, tanhf(__fdiv_rn(x[i], cap)));
    }
}

}  // namespace b200

#endif  // B200_NORM_CHAINS_CUH
