// stream_ops.cuh -- the remaining row-parallel kernels of the reference's gpu_ops module: hyper-connections and PLE
// (src/gpu_ops.hip:322-476: the residual is hc streams of n values per token, rows r = t * hc + c), the MTP head's
// input, and Mamba-2's gated group norm (:763-792).
//   hc_norm      res_out[r] = res_in[r] + cur[t] * (2 * sigmoid(inject[r] / hc)) when cur is given;
//                y[r] = RMSNorm(that) * w[c * n ..]
//   hc_lowrank   out[t] = SiLU(lo[t] / hc), rows of n values zero-padded to np
//   hc_mix       out[t] = (sum over c, in order, of xn[r] * sigmoid(gate[r])) / hc
//   mtp_concat   out[r] = [e[t] | h[r]]
//   ple_gate     per stream: s = (RMSNorm(key[r]) * wk) . (RMSNorm(res[r]) * wq) / sqrt(n);
//                g = sigmoid(sgn(s) * sqrt(max(|s|, 1e-6))); gated[r] = value[t] * g; normed[r] = RMSNorm(gated[r]) * wc
//   mamba_gnorm  v = y * SiLU(z) over a group of d_inner / n_group values; out = RMSNorm(v) * w
// Arithmetic as everywhere in this library: every fp32 product and sum rounded on its own in the order the reference
// writes them, sums of squares and dot products carried in double, 1/rms as (float)(1 / sqrt(ss / n + eps)),
// sigmoid and SiLU with the accurate expf and an IEEE division (the reference's kernels use the fast __expf; its CPU
// graph, llama.cpp's, uses expf). Rows of the norm kernels are exactly blockDim.x * VPT 16-byte vectors, one CTA per
// row, each value read once and written once per output.

#ifndef B200_STREAM_OPS_CUH
#define B200_STREAM_OPS_CUH

#include "common.cuh"
#include "norm_chains.cuh"

namespace b200 {

__device__ __forceinline__ float sigmoid_f(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float silu_f(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }

template <int VPT>
__global__ void __launch_bounds__(512)
k_hc_norm(const float* res_in, float* res_out, const float* cur, const float* inject, const float* w, float* y, int n,
          int hc, long long rows, float eps) {
    __shared__ double part[2][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const size_t row_vecs = (size_t)tpr * VPT;
    const double inv_n = 1.0 / (double)n;
    const float inv_hc = __fdiv_rn(1.0f, (float)hc);
    int flip = 0;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x, flip ^= 1) {
        const long long t = r / hc;
        const int c = (int)(r - t * hc);
        const size_t off = (size_t)r * row_vecs + l;
        f2 v[VPT][2];
        uint4 ru[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(res_in) + off + j * tpr), v[j]);
            if (cur) ru[j] = ld_stream(reinterpret_cast<const uint4*>(cur) + (size_t)t * row_vecs + l + j * tpr);
        }
        if (cur) {   // uniform
            const float wt = __fmul_rn(2.0f, sigmoid_f(__fmul_rn(__ldg(inject + r), inv_hc)));
            const f2 wt2 = pk2(wt, wt);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                f2 u[2];
                Io2<float>::unpack(ru[j], u);
                v[j][0] = add_rounded(v[j][0], mul2(u[0], wt2));
                v[j][1] = add_rounded(v[j][1], mul2(u[1], wt2));
                st_stream(reinterpret_cast<uint4*>(res_out) + off + j * tpr, Io2<float>::pack(v[j]));
            }
        }
        const float inv = inv_rms(cta_sum(row_sumsq<VPT>(v), part[flip]), inv_n, eps);
        const f2 inv2 = pk2(inv, inv);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 g[2], o[2];
            gamma_pair(w, (size_t)c * row_vecs + l + (size_t)j * tpr, g);
            o[0] = mul2(mul2(v[j][0], inv2), g[0]);
            o[1] = mul2(mul2(v[j][1], inv2), g[1]);
            st_stream(reinterpret_cast<uint4*>(y) + off + j * tpr, Io2<float>::pack(o));
        }
    }
}

// out [T][np]: SiLU(lo[t][k] * scale) for k < n, 0 for n <= k < np
__global__ void __launch_bounds__(256)
k_hc_lowrank(const float* lo, float* out, int n, int np, long long T, float scale) {
    const long long total = T * np;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / np;
        const int k = (int)(i - t * np);
        out[i] = k < n ? silu_f(__fmul_rn(lo[t * n + k], scale)) : 0.0f;
    }
}

// VEC: n a multiple of 4 and 16-byte aligned bases
template <bool VEC>
__global__ void __launch_bounds__(256)
k_hc_mix(const float* xn, const float* gate, float* out, int n, int hc, long long T) {
    const int per_row = VEC ? n / 4 : n, W = VEC ? 4 : 1;
    const long long total = T * per_row;
    const float inv_hc = __fdiv_rn(1.0f, (float)hc);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per_row;
        const int k = (int)(i - t * per_row) * W;
        const size_t base = (size_t)t * hc * n + k;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int c = 0; c < hc; ++c) {
            float x[4], g[4];
            if (VEC) {
                Io<float>::unpack(ld_stream(xn + base + (size_t)c * n), x);
                Io<float>::unpack(ld_stream(gate + base + (size_t)c * n), g);
            } else {
                x[0] = xn[base + (size_t)c * n];
                g[0] = gate[base + (size_t)c * n];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (e < W) {
                    const float p = __fmul_rn(x[e], sigmoid_f(g[e]));
                    acc[e] = c == 0 ? p : __fadd_rn(acc[e], p);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = __fmul_rn(acc[e], inv_hc);
        if (VEC) st_stream(out + t * (long long)n + k, Io<float>::pack(acc));
        else out[t * (long long)n + k] = acc[0];
    }
}

// out [T * hc][2 n]: e[t] then h[r]. VEC: n a multiple of 4 and aligned bases
template <bool VEC>
__global__ void __launch_bounds__(256)
k_mtp_concat(const float* e, const float* h, float* out, int n, int hc, long long rows) {
    const int per_row = VEC ? (2 * n) / 4 : 2 * n, W = VEC ? 4 : 1;
    const long long total = rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / per_row;
        const int k = (int)(i - r * per_row) * W;
        const float* src = k < n ? e + (r / hc) * n + k : h + r * n + (k - n);
        if (VEC) st_stream(out + r * 2 * n + k, ld_stream(src));
        else out[r * 2 * n + k] = *src;
    }
}

template <int VPT>
__global__ void __launch_bounds__(512)
k_ple_gate(const float* key, const float* value, const float* res, const float* wk, const float* wq, const float* wc,
           float* gated, float* normed, int n, int hc, long long T, float eps) {
    __shared__ double part[4][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const size_t row_vecs = (size_t)tpr * VPT;
    const double inv_n = 1.0 / (double)n;
    const float inv_sqrt_n = __fdiv_rn(1.0f, __fsqrt_rn((float)n));
    for (long long t = blockIdx.x; t < T; t += gridDim.x) {
        f2 val[VPT][2];
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(value) + (size_t)t * row_vecs + l + j * tpr), val[j]);
        for (int c = 0; c < hc; ++c) {
            const size_t off = ((size_t)t * hc + c) * row_vecs + l, woff = (size_t)c * row_vecs + l;
            f2 kx[VPT][2], qx[VPT][2];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(key) + off + j * tpr), kx[j]);
                Io2<float>::unpack(ld_stream(reinterpret_cast<const uint4*>(res) + off + j * tpr), qx[j]);
            }
            const float ik = inv_rms(cta_sum(row_sumsq<VPT>(kx), part[0]), inv_n, eps);
            const float iq = inv_rms(cta_sum(row_sumsq<VPT>(qx), part[1]), inv_n, eps);
            const f2 ik2 = pk2(ik, ik), iq2 = pk2(iq, iq);
            double d0 = 0.0, d1 = 0.0;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                f2 gk[2], gq[2];
                gamma_pair(wk, woff + (size_t)j * tpr, gk);
                gamma_pair(wq, woff + (size_t)j * tpr, gq);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    float p0, p1;
                    upk2(mul2(mul2(mul2(kx[j][k], ik2), gk[k]), mul2(mul2(qx[j][k], iq2), gq[k])), p0, p1);
                    d0 += (double)p0;
                    d1 += (double)p1;
                }
            }
            const float s = __fmul_rn((float)cta_sum(d0 + d1, part[2]), inv_sqrt_n);
            const float mag = __fsqrt_rn(fmaxf(fabsf(s), 1e-6f));
            const float g = sigmoid_f(__fmul_rn(s > 0.0f ? 1.0f : (s < 0.0f ? -1.0f : 0.0f), mag));
            const f2 g2 = pk2(g, g);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                kx[j][0] = mul2(val[j][0], g2);
                kx[j][1] = mul2(val[j][1], g2);
                st_stream(reinterpret_cast<uint4*>(gated) + off + j * tpr, Io2<float>::pack(kx[j]));
            }
            const float ig = inv_rms(cta_sum(row_sumsq<VPT>(kx), part[3]), inv_n, eps);
            const f2 ig2 = pk2(ig, ig);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                f2 gc[2], o[2];
                gamma_pair(wc, woff + (size_t)j * tpr, gc);
                o[0] = mul2(mul2(kx[j][0], ig2), gc[0]);
                o[1] = mul2(mul2(kx[j][1], ig2), gc[1]);
                st_stream(reinterpret_cast<uint4*>(normed) + off + j * tpr, Io2<float>::pack(o));
            }
        }
    }
}

// A CTA of gs / 8 threads per (token, group): two vectors per thread
__global__ void __launch_bounds__(128)
k_mamba_gnorm(const float* y, const float* zx, long long ld, const float* w, float* out, int d_inner, int n_group,
              long long T, float eps) {
    __shared__ double part[2][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const int gs = d_inner / n_group;
    const double inv_n = 1.0 / (double)gs;
    const long long rows = T * n_group;
    int flip = 0;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x, flip ^= 1) {
        const long long t = r / n_group;
        const int g = (int)(r - t * n_group);
        const float* yr = y + t * d_inner + (long long)g * gs;
        const float* zr = zx + t * ld + (long long)g * gs;
        f2 v[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float a[4], z[4];
            Io<float>::unpack(ld_stream(yr + (l + j * tpr) * 4), a);
            Io<float>::unpack(ld_stream(zr + (l + j * tpr) * 4), z);
#pragma unroll
            for (int e = 0; e < 4; ++e) a[e] = __fmul_rn(a[e], silu_f(z[e]));
            v[j][0] = pk2(a[0], a[1]);
            v[j][1] = pk2(a[2], a[3]);
        }
        const float inv = inv_rms(cta_sum(row_sumsq<2>(v), part[flip]), inv_n, eps);
        const f2 inv2 = pk2(inv, inv);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            f2 gam[2], o[2];
            gamma_pair(w + (long long)g * gs, (size_t)l + (size_t)j * tpr, gam);
            o[0] = mul2(mul2(v[j][0], inv2), gam[0]);
            o[1] = mul2(mul2(v[j][1], inv2), gam[1]);
            st_stream(reinterpret_cast<uint4*>(out + t * d_inner + (long long)g * gs) + l + j * tpr, Io2<float>::pack(o));
        }
    }
}

}  // namespace b200

#endif  // B200_STREAM_OPS_CUH
