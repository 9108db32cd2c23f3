// window_ops.cuh -- the kernels of the reference's gpu_ops module that look back over earlier tokens
// (src/gpu_ops.hip:476-512 ple_conv, :679-760 mamba_conv / mamba_conv_state / mamba_scan):
//   mamba_conv  out[t][c] = SiLU(sum_i window_i * w[c][i] + bias[c]): the window is the d_conv - 1 inputs before token
//               t (rows of zx at x_off, or the conv state [c][d_conv - 1] for positions before the batch) and token
//               t's own, oldest first; then the state becomes the batch's last d_conv - 1 inputs
//   ple_conv    res[t][ch] += gated[t][ch] + SiLU(sum_k x[t - (K - 1 - k) dil][ch] * w[ch][k]), x = normed with the
//               (K - 1) dil rows of state before it, fp16 taps; the state is advanced; optionally the states after the
//               first tokens are kept (rollback points of a speculative pass)
//   mamba_scan  Mamba-2's selective scan: per head h and dim i a state of 128 values; per token dt = softplus(dt_t +
//               dt_b[h]), dA = exp(dt A[h]), s = s dA + B (x dt), y = sum_j s_j C_j + x D[h]
// The two convolutions read only inputs, so every (token, channel) output is independent: one thread per four
// channels of a token, grid-stride, and a second small launch that advances the state once all outputs have read the
// old one (same stream). The scan is a true recurrence over the tokens; its rows (head, dim) are independent, so a
// CTA takes 16 of a head's 64 dims (four CTAs per head, where the reference has one) to spread a model's heads over
// more SMs. Sums run in the reference's order, each product and sum rounded on its own except the explicit fused
// multiply-add of the scan's output sum; SiLU / softplus / exp use the accurate library functions.

#ifndef B200_WINDOW_OPS_CUH
#define B200_WINDOW_OPS_CUH

#include "common.cuh"
#include "stream_ops.cuh"

namespace b200 {

#define MAMBA_DS 128   // state values per (head, dim)
#define MAMBA_P 64     // dims per head
#define MAMBA_MAXC 8   // taps of the Mamba conv

struct MidStates {  // the reference's deltanet_mid_states by value: p[j], when set, receives the state after token j
    float* p[3];
};

// W: channels per thread (4: conv_dim, ld, x_off multiples of 4 and aligned bases; else 1)
template <int W>
__global__ void __launch_bounds__(256)
k_mamba_conv(const float* zx, long long ld, int x_off, const float* conv_state, const float* w, const float* bias,
             float* out, int conv_dim, int d_conv, long long T) {
    const int per_row = conv_dim / W, ns = d_conv - 1;
    const long long total = T * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per_row;
        const int c = (int)(i - t * per_row) * W;
        float s[W];
#pragma unroll
        for (int e = 0; e < W; ++e) s[e] = 0.0f;
        for (int k = 0; k <= ns; ++k) {
            const long long tt = t - ns + k;
            float h[4];
            if (tt >= 0) {
                if (W == 4) Io<float>::unpack(ld_stream(zx + tt * ld + x_off + c), h);
                else h[0] = zx[tt * ld + x_off + c];
            } else {
#pragma unroll
                for (int e = 0; e < W; ++e) h[e] = conv_state[(size_t)(c + e) * ns + ns + tt];
            }
#pragma unroll
            for (int e = 0; e < W; ++e) s[e] = __fadd_rn(s[e], __fmul_rn(h[e], __ldg(w + (size_t)(c + e) * d_conv + k)));
        }
        float o[4];
#pragma unroll
        for (int e = 0; e < W; ++e) o[e] = silu_f(__fadd_rn(s[e], __ldg(bias + c + e)));
        if (W == 4) st_stream(out + t * conv_dim + c, Io<float>::pack(o));
        else out[t * conv_dim + c] = o[0];
    }
}

// Channel c's conv state after T tokens: the last d_conv - 1 inputs, oldest first
__device__ __forceinline__ void mamba_conv_state_channel(const float* zx, long long ld, int x_off, float* conv_state, int c,
                                                         int d_conv, long long T) {
    const int ns = d_conv - 1;
    float* st = conv_state + (size_t)c * ns;
    float h[MAMBA_MAXC];
    for (int i = 0; i < ns; ++i) {
        const long long tt = T - ns + i;
        h[i] = tt >= 0 ? zx[tt * ld + x_off + c] : st[i + T];
    }
    for (int i = 0; i < ns; ++i) st[i] = h[i];
}

__global__ void __launch_bounds__(256)
k_mamba_conv_state(const float* zx, long long ld, int x_off, float* conv_state, int conv_dim, int d_conv, long long T) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < conv_dim) mamba_conv_state_channel(zx, ld, x_off, conv_state, c, d_conv, T);
}

template <int W>
__global__ void __launch_bounds__(256)
k_ple_conv(const float* normed, const float* gated, float* res, const float* state, const __half* w, int m, long long T,
           int K, int dil) {
    const int per_row = m / W, H = (K - 1) * dil;
    const long long total = T * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per_row;
        const int ch = (int)(i - t * per_row) * W;
        float acc[4];
        for (int k = 0; k < K; ++k) {
            const long long j = t - (long long)(K - 1 - k) * dil;
            const float* src = j >= 0 ? normed + j * m + ch : state + (H + j) * m + ch;
            float x[4];
            if (W == 4) Io<float>::unpack(ld_stream(src), x);
            else x[0] = *src;
#pragma unroll
            for (int e = 0; e < W; ++e) {
                const float term = __fmul_rn(x[e], __half2float(w[(size_t)(ch + e) * K + k]));
                acc[e] = k == 0 ? term : __fadd_rn(acc[e], term);
            }
        }
        const size_t at = (size_t)t * m + ch;
        float g[4], r[4];
        if (W == 4) {
            Io<float>::unpack(ld_stream(gated + at), g);
            Io<float>::unpack(ld_stream(res + at), r);
        } else {
            g[0] = gated[at];
            r[0] = res[at];
        }
#pragma unroll
        for (int e = 0; e < W; ++e) r[e] = __fadd_rn(r[e], __fadd_rn(g[e], silu_f(acc[e])));
        if (W == 4) st_stream(res + at, Io<float>::pack(r));
        else res[at] = r[0];
    }
}

// The states after the first tokens, then the state after the batch: row i of a state is row (tokens seen + i) of
// [old state rows | normed rows]. One thread per channel; ascending i only reads rows above i of the old state.
__device__ __forceinline__ void ple_conv_state_channel(const float* normed, float* state, int m, long long T, int K, int dil,
                                                       const MidStates& mid, int ch) {
    const int H = (K - 1) * dil;
    for (int j = 0; j < 3 && j < T - 1; ++j)
        if (mid.p[j])
            for (int i = 0; i < H; ++i) {
                const int src = j + 1 + i;
                mid.p[j][(size_t)i * m + ch] = src < H ? state[(size_t)src * m + ch] : normed[(size_t)(src - H) * m + ch];
            }
    for (int i = 0; i < H; ++i) {
        const long long src = T + i;
        state[(size_t)i * m + ch] = src < H ? state[(size_t)src * m + ch] : normed[(size_t)(src - H) * m + ch];
    }
}

__global__ void __launch_bounds__(256)
k_ple_conv_state(const float* normed, float* state, int m, long long T, int K, int dil, MidStates mid) {
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch < m) ple_conv_state_channel(normed, state, m, T, K, dil, mid, ch);
}

// The recurrence of one thread: dim i of head h, state values 32 q .. 32 q + 31 (the four threads of a dim are four
// neighbouring lanes)
__device__ __forceinline__ void mamba_scan_thread(float* state, const float* xbc, const float* zx, long long ld, int dt_off,
                                                  const float* dt_b, const float* A, const float* D, float* y, int n_head,
                                                  int d_inner, int n_group, long long T, int h, int i, int q) {
    const int g = h / (n_head / n_group), conv_dim = d_inner + 2 * n_group * MAMBA_DS;
    float* st = state + ((size_t)h * MAMBA_P + i) * MAMBA_DS + 32 * q;
    float s[32];
#pragma unroll
    for (int j = 0; j < 32; j += 4) Io<float>::unpack(*reinterpret_cast<const uint4*>(st + j), s + j);
    const float a = A[h], dh = D[h], db = dt_b[h];
    for (long long t = 0; t < T; ++t) {
        const float* row = xbc + t * conv_dim;
        const float dv = __fadd_rn(zx[t * ld + dt_off + h], db);
        const float sp = dv > 20.0f ? dv : log1pf(expf(dv));
        const float dA = expf(__fmul_rn(sp, a));
        const float x = row[h * MAMBA_P + i], xdt = __fmul_rn(x, sp);
        const float* Bp = row + d_inner + g * MAMBA_DS + 32 * q;
        const float* Cp = row + d_inner + (n_group + g) * MAMBA_DS + 32 * q;
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            float b[4], c[4];
            Io<float>::unpack(__ldg(reinterpret_cast<const uint4*>(Bp + j)), b);
            Io<float>::unpack(__ldg(reinterpret_cast<const uint4*>(Cp + j)), c);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[j + e] = __fadd_rn(__fmul_rn(s[j + e], dA), __fmul_rn(b[e], xdt));
                acc = fmaf(s[j + e], c[e], acc);
            }
        }
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        if (q == 0) y[t * d_inner + h * MAMBA_P + i] = __fadd_rn(acc, __fmul_rn(x, dh));
    }
#pragma unroll
    for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(st + j) = Io<float>::pack(s + j);
}

// CTA of 64 threads: dims 16 part .. 16 part + 15 of head h, four threads per dim
__global__ void __launch_bounds__(64)
k_mamba_scan(float* state, const float* xbc, const float* zx, long long ld, int dt_off, const float* dt_b, const float* A,
             const float* D, float* y, int n_head, int d_inner, int n_group, long long T) {
    mamba_scan_thread(state, xbc, zx, ld, dt_off, dt_b, A, D, y, n_head, d_inner, n_group, T, blockIdx.x >> 2,
                      (blockIdx.x & 3) * 16 + (threadIdx.x >> 2), threadIdx.x & 3);
}

}  // namespace b200

#endif  // B200_WINDOW_OPS_CUH
