// rope_f16.cuh -- rotate-half RoPE on fp16 rows with host-built fp32 cos / sin tables, the math of the reference's
// rope_rotate_half kernel (src/rope_embedding.hip:18-37) and of its test's CPU loop (tests/rope_verify.cpp:84-93):
//   y[r][i] = x[r][i] c - x[r][i+H] s;  y[r][i+H] = x[r][i+H] c + x[r][i] s,  c = ctab[r][i], s = stab[r][i],
// fp32 products and sums each rounded (no fused multiply-add), one rounding to fp16. y may be x: a thread reads both
// halves of its pairs before it writes them. Per row 2 * 2H * 2 bytes of activations and 2 * H * 4 bytes of tables.

#ifndef B200_ROPE_F16_CUH
#define B200_ROPE_F16_CUH

#include "common.cuh"

namespace b200 {

// half_dim % 8 == 0, all bases 16-byte aligned: a thread takes 8 pairs (one vector of each half)
__global__ void __launch_bounds__(256)
k_rope_rotate_half_f16_vec(const __half* x, const float* ctab, const float* stab, __half* y, int n_rows, int H) {
    const int hv = H / 8;
    const long long total = (long long)n_rows * hv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / hv;
        const int c0 = (int)(i - r * hv) * 8;
        const __half* xr = x + (size_t)r * 2 * H;
        __half* yr = y + (size_t)r * 2 * H;
        const uint4 rlo = ld_stream(xr + c0), rhi = ld_stream(xr + H + c0);
        float lo[8], hi[8], c[8], s[8], olo[8], ohi[8];
        Io<__half>::unpack(rlo, lo);
        Io<__half>::unpack(rhi, hi);
        Io<float>::unpack(ld_stream(ctab + (size_t)r * H + c0), c);
        Io<float>::unpack(ld_stream(ctab + (size_t)r * H + c0 + 4), c + 4);
        Io<float>::unpack(ld_stream(stab + (size_t)r * H + c0), s);
        Io<float>::unpack(ld_stream(stab + (size_t)r * H + c0 + 4), s + 4);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            olo[e] = __fsub_rn(__fmul_rn(lo[e], c[e]), __fmul_rn(hi[e], s[e]));
            ohi[e] = __fadd_rn(__fmul_rn(hi[e], c[e]), __fmul_rn(lo[e], s[e]));
        }
        st_stream(yr + c0, Io<__half>::pack(olo));
        st_stream(yr + H + c0, Io<__half>::pack(ohi));
    }
}

// any half_dim and alignment: one pair per thread and step
__global__ void __launch_bounds__(256)
k_rope_rotate_half_f16(const __half* x, const float* ctab, const float* stab, __half* y, int n_rows, int H) {
    const long long total = (long long)n_rows * H;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / H;
        const int c0 = (int)(i - r * H);
        const float lo = __half2float(x[(size_t)r * 2 * H + c0]), hi = __half2float(x[(size_t)r * 2 * H + H + c0]);
        const float c = ctab[i], s = stab[i];
        y[(size_t)r * 2 * H + c0] = __float2half_rn(__fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)));
        y[(size_t)r * 2 * H + H + c0] = __float2half_rn(__fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s)));
    }
}

}  // namespace b200

#endif  // B200_ROPE_F16_CUH
