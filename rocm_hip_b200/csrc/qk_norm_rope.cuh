// qk_norm_rope.cuh -- per-head q/k RMSNorm fused with NeoX rotary embedding, the B200 kernels behind
// gpu_qk_norm_rope. Math of the reference's norm_rope<D> (src/attention.hip:212-236) as its CPU references state it
// (qwen_rmsnorm + qwen_rope_neox, src/qwen_ops.cpp:8-24; qk_ref, tests/forward_verify.cpp:835-853): per head
//   x *= rsqrt(mean(x^2) + eps) * w[d];  pairs (i, i + n_rot/2), i < rot_pairs, rotate by theta_i = pos * base^(-2i/n_rot)
//   (divided by ff[i] when frequency factors are given); dims >= n_rot and pairs >= rot_pairs stay as they are.
// Unlike the reference kernel, which forms theta in fp32 (tested to 1e-3 at position 2499), the angle here is the
// double product pos * inv_freq[i] with inv_freq built on the host by the CPU reference's own expression, and
// cos / sin are evaluated in double and rounded once: that is what holds 1e-5 at positions in the hundreds of thousands.
//
// One CTA pass handles one token: all of its n_q + n_kv heads. A head of D values is NV = D / VE 16-byte vectors,
// owned by NV / (2 PPT) threads. Each thread owns PPT pairs of vectors; a rotating thread owns the vector of a
// rotation pair's low half and the vector of its high half, so the rotation needs no exchange, the row is read
// once and written once (2 D s bytes per head), and the sum of squares is a shuffle reduction inside the head's lanes.
// The token's cos / sin (n_rot / 2 each) are computed once by the first threads, while the loads are in flight, and
// shared by all heads through shared memory.

#ifndef B200_QK_NORM_ROPE_CUH
#define B200_QK_NORM_ROPE_CUH

#include "common.cuh"

namespace b200 {

#define B200_MAX_ROT_PAIRS 256

// Angle multipliers of the rotation pairs, passed by value (2 KB of kernel parameters)
struct RopeFreq {
    double inv_freq[B200_MAX_ROT_PAIRS];
};

struct QkArgs {
    const void* qfull;   // [T][n_q * q_stride]
    const void* k;       // [T][n_kv * D]
    void* q_out;         // [T][n_q * D]
    void* k_out;         // [T][n_kv * D]
    const float* q_norm; // [D] or NULL
    const float* k_norm; // [D] or NULL
    const float* ff;     // [n_rot / 2] or NULL
    const int* positions;// [T] or NULL (then pos0 + t)
    int n_q, n_kv, D, q_stride;
    int n_rot, rot_pairs;  // rot_pairs <= n_rot / 2
    int pos0, do_norm;
    long long T;
    float eps;
};

// cos / sin of this token's angles into cs[pair] = (cos, sin); threads 0 .. rot_pairs-1 take one pair each
// (in steps of blockDim.x)
__device__ __forceinline__ void token_cos_sin(float2* cs, const QkArgs& a, const RopeFreq& fr, long long t) {
    if ((int)threadIdx.x >= a.rot_pairs) return;
    const int pos = a.positions ? a.positions[t] : a.pos0 + (int)t;
    for (int i = threadIdx.x; i < a.rot_pairs; i += blockDim.x) {
        double theta = (double)pos * fr.inv_freq[i];
        if (a.ff) theta /= (double)a.ff[i];
        double s, c;
        sincos(theta, &s, &c);
        cs[i] = make_float2((float)c, (float)s);
    }
}

// PPT: pairs of vectors per thread. Threads per head tph = D / VE / (2 PPT), a power of two <= 32.
template <typename IO, int PPT>
__global__ void __launch_bounds__(1024)
k_qk_norm_rope(const QkArgs a, const __grid_constant__ RopeFreq fr) {
    constexpr int VE = Io<IO>::VE;
    __shared__ float2 cs[2][B200_MAX_ROT_PAIRS];
    const int D = a.D, NV = D / VE, tph = NV / (2 * PPT);
    const int R = a.n_rot / VE;      // vectors in the rotary part
    const int P = R / 2;             // pairs of vectors (low half, high half)
    const int heads = a.n_q + a.n_kv;
    const int heads_per_pass = blockDim.x / tph;
    const int l = threadIdx.x % tph, hslot = threadIdx.x / tph;

    // this thread's vector slots within a head: slot s < P pairs vector s with s + P; the rest pair up neighbours
    int vlo[PPT], vhi[PPT];
    bool rot[PPT];
#pragma unroll
    for (int p = 0; p < PPT; ++p) {
        const int s = l + p * tph;  // 0 .. NV/2-1
        rot[p] = s < P;
        vlo[p] = rot[p] ? s : R + 2 * (s - P);
        vhi[p] = rot[p] ? s + P : R + 2 * (s - P) + 1;
    }

    int flip = 0;
    for (long long t = blockIdx.x; t < a.T; t += gridDim.x, flip ^= 1) {
        const IO* qrow = static_cast<const IO*>(a.qfull) + (size_t)t * a.n_q * a.q_stride;
        const IO* krow = static_cast<const IO*>(a.k) + (size_t)t * a.n_kv * D;
        IO* qo = static_cast<IO*>(a.q_out) + (size_t)t * a.n_q * D;
        IO* ko = static_cast<IO*>(a.k_out) + (size_t)t * a.n_kv * D;
        bool tables_done = false;
        for (int h0 = 0; h0 < heads; h0 += heads_per_pass) {
            const int h = h0 + hslot;
            const bool live = h < heads;
            const bool isq = h < a.n_q;
            const IO* src = isq ? qrow + (size_t)h * a.q_stride : krow + (size_t)(h - a.n_q) * D;
            IO* dst = isq ? qo + (size_t)h * D : ko + (size_t)(h - a.n_q) * D;
            const float* gamma = isq ? a.q_norm : a.k_norm;
            uint4 rlo[PPT], rhi[PPT];
            if (live) {
#pragma unroll
                for (int p = 0; p < PPT; ++p) {
                    rlo[p] = ld_stream(reinterpret_cast<const uint4*>(src) + vlo[p]);
                    rhi[p] = ld_stream(reinterpret_cast<const uint4*>(src) + vhi[p]);
                }
            }
            if (!tables_done) {  // uniform over the CTA
                token_cos_sin(cs[flip], a, fr, t);
                __syncthreads();
                tables_done = true;
            }
            float lo[PPT][VE], hi[PPT][VE];
            float ss = 0.0f;
            if (live) {
#pragma unroll
                for (int p = 0; p < PPT; ++p) {
                    Io<IO>::unpack(rlo[p], lo[p]);
                    Io<IO>::unpack(rhi[p], hi[p]);
#pragma unroll
                    for (int e = 0; e < VE; ++e) ss = fmaf(lo[p][e], lo[p][e], ss);
#pragma unroll
                    for (int e = 0; e < VE; ++e) ss = fmaf(hi[p][e], hi[p][e], ss);
                }
            }
            if (a.do_norm) {  // uniform
                const float tot = group_sum(ss, tph);
                const float inv = inv_rms(tot, D, a.eps);
                if (live) {
#pragma unroll
                    for (int p = 0; p < PPT; ++p) {
                        float gl[VE], gh[VE];
                        load_gamma<VE, float>(gamma, vlo[p] * VE, gl);
                        load_gamma<VE, float>(gamma, vhi[p] * VE, gh);
#pragma unroll
                        for (int e = 0; e < VE; ++e) {
                            lo[p][e] = __fmul_rn(__fmul_rn(lo[p][e], inv), gl[e]);
                            hi[p][e] = __fmul_rn(__fmul_rn(hi[p][e], inv), gh[e]);
                        }
                    }
                }
            }
            if (live) {
#pragma unroll
                for (int p = 0; p < PPT; ++p) {
                    if (rot[p]) {
                        const int i0 = vlo[p] * VE;  // first pair index of this vector
#pragma unroll
                        for (int e = 0; e < VE; ++e) {
                            if (i0 + e < a.rot_pairs) {
                                const float2 c = cs[flip][i0 + e];
                                const float x0 = lo[p][e], x1 = hi[p][e];
                                // src/qwen_ops.cpp:21-22: x0 c - x1 s and x0 s + x1 c, each product rounded
                                lo[p][e] = __fsub_rn(__fmul_rn(x0, c.x), __fmul_rn(x1, c.y));
                                hi[p][e] = __fadd_rn(__fmul_rn(x0, c.y), __fmul_rn(x1, c.x));
                            }
                        }
                    }
                    st_stream(reinterpret_cast<uint4*>(dst) + vlo[p], Io<IO>::pack(lo[p]));
                    st_stream(reinterpret_cast<uint4*>(dst) + vhi[p], Io<IO>::pack(hi[p]));
                }
            }
        }
    }
}

// Any head size, rotary width and alignment: one CTA pass per token, heads one after the other, the normalised head
// staged in shared memory so that a value can read its rotation partner (the reference kernel's own scheme).
// D <= 1024.
template <typename IO>
__global__ void __launch_bounds__(128)
k_qk_norm_rope_generic(const QkArgs a, const __grid_constant__ RopeFreq fr) {
    __shared__ float2 cs[B200_MAX_ROT_PAIRS];
    __shared__ float v[1024];
    __shared__ float part[2][32];
    const int D = a.D, half = a.n_rot / 2, heads = a.n_q + a.n_kv;
    int flip = 0;
    for (long long t = blockIdx.x; t < a.T; t += gridDim.x) {
        __syncthreads();  // the previous token's tables and head are no longer read
        token_cos_sin(cs, a, fr, t);
        for (int h = 0; h < heads; ++h) {
            const bool isq = h < a.n_q;
            const IO* src = isq ? static_cast<const IO*>(a.qfull) + ((size_t)t * a.n_q + h) * a.q_stride
                                : static_cast<const IO*>(a.k) + ((size_t)t * a.n_kv + (h - a.n_q)) * D;
            IO* dst = isq ? static_cast<IO*>(a.q_out) + ((size_t)t * a.n_q + h) * D
                          : static_cast<IO*>(a.k_out) + ((size_t)t * a.n_kv + (h - a.n_q)) * D;
            const float* gamma = isq ? a.q_norm : a.k_norm;
            float ss = 0.0f;
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                const float x = Io<IO>::load1(src + d);
                v[d] = x;
                ss = fmaf(x, x, ss);
            }
            float inv = 1.0f;
            if (a.do_norm) {
                inv = inv_rms(cta_sum(ss, part[flip]), D, a.eps);
                flip ^= 1;
                for (int d = threadIdx.x; d < D; d += blockDim.x)  // this thread's own values
                    v[d] = __fmul_rn(__fmul_rn(v[d], inv), gamma1(gamma, d));
            }
            __syncthreads();
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                float x = v[d];
                const int i = d < half ? d : d - half;
                if (d < a.n_rot && i < a.rot_pairs) {
                    const float2 c = cs[i];
                    const float x0 = v[i], x1 = v[i + half];
                    x = d < half ? __fsub_rn(__fmul_rn(x0, c.x), __fmul_rn(x1, c.y))
                                 : __fadd_rn(__fmul_rn(x0, c.y), __fmul_rn(x1, c.x));
                }
                Io<IO>::store1(dst + d, x);
            }
            __syncthreads();  // v is rewritten by the next head
        }
    }
}

}  // namespace b200

#endif  // B200_QK_NORM_ROPE_CUH
