// rmsnorm.cuh -- residual add + RMSNorm over rows, the B200 kernels behind gpu_add_rmsnorm and its bf16 / fp16
// siblings. Math of the reference's add_rmsnorm / add_rmsnorm_rows (src/gpu_ops.hip:24-101):
//   v = x_in + add (when add is set; v is stored to x_out), y = v * rsqrt(mean(v^2) + eps) * w, two multiplies
//   left to right as src/qwen_ops.cpp:12 and src/gpu_ops.hip:52 evaluate them.
// For 16-bit rows the arithmetic is fp32 and the norm is taken of the value as stored in x_out (rounded), so a
// fused call gives the bits of a separate add followed by a norm.
//
// Layout: rows [T][n] contiguous. A row is read exactly once with 16-byte loads into registers (VPT vectors per
// thread), reduced, scaled and written with 16-byte stores: 2 n s bytes per row without add, 4 n s with (s = bytes
// per value), which is the algorithmic minimum. Two shapes:
//   * rows of up to 32 * VPT vectors: a lane group of tpr <= 32 threads per row, several rows per CTA, shuffles only;
//   * wider rows: one CTA of tpr threads per row (tpr a multiple of 32), one shared-memory exchange per row.
// The launcher picks (tpr, VPT) from n and the storage type alone, never from T or the grid, so the summation
// order of a row is fixed. CTAs walk rows with a grid stride, which lets the gammas stay in registers.

#ifndef B200_RMSNORM_CUH
#define B200_RMSNORM_CUH

#include "common.cuh"

namespace b200 {

// CTA_ROW = false: lane groups of tpr threads (power of two <= 32), blockDim.x / tpr rows per pass.
// CTA_ROW = true : the whole CTA (tpr == blockDim.x) works on one row per pass.
template <typename IO, typename WT, int VPT, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 1024 : 256)
k_add_rmsnorm(const IO* x_in, const IO* add, IO* x_out, const WT* w, IO* y, int n, long long T, float eps, int tpr) {
    constexpr int VE = Io<IO>::VE;
    __shared__ float part[2][32];
    const int nvec = n / VE;
    const int l = CTA_ROW ? (int)threadIdx.x : (int)threadIdx.x % tpr;
    const int g = CTA_ROW ? 0 : (int)threadIdx.x / tpr;
    const int rows_per_pass = CTA_ROW ? 1 : (int)blockDim.x / tpr;

    float gam[VPT][VE];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int vi = l + j * tpr;
        if (vi < nvec) load_gamma<VE, WT>(w, vi * VE, gam[j]);
    }

    int flip = 0;
    // every thread of a warp runs the same number of passes (shuffles need all lanes); rows past T are masked
    for (long long base = (long long)blockIdx.x * rows_per_pass; base < T; base += (long long)gridDim.x * rows_per_pass) {
        const long long row = base + g;
        const bool live = row < T;
        const size_t off = (size_t)(live ? row : 0) * (size_t)n;
        const uint4* px = reinterpret_cast<const uint4*>(x_in + off);
        const uint4* pa = add ? reinterpret_cast<const uint4*>(add + off) : nullptr;
        uint4* po = reinterpret_cast<uint4*>(x_out + off);
        uint4* py = reinterpret_cast<uint4*>(y + off);

        uint4 rx[VPT], ra[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int vi = l + j * tpr;
            if (live && vi < nvec) {
                rx[j] = ld_stream(px + vi);
                if (pa) ra[j] = ld_stream(pa + vi);
            }
        }
        float v[VPT][VE];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int vi = l + j * tpr;
            if (live && vi < nvec) {
                Io<IO>::unpack(rx[j], v[j]);
                if (pa) {
                    float a[VE];
                    Io<IO>::unpack(ra[j], a);
#pragma unroll
                    for (int e = 0; e < VE; ++e) v[j][e] = __fadd_rn(v[j][e], a[e]);
                    const uint4 packed = Io<IO>::pack(v[j]);
                    st_stream(po + vi, packed);
                    if (sizeof(IO) < 4) Io<IO>::unpack(packed, v[j]);  // the norm sees the stored value
                }
#pragma unroll
                for (int e = 0; e < VE; ++e) ss = fmaf(v[j][e], v[j][e], ss);
            }
        }
        const float tot = CTA_ROW ? cta_sum(ss, part[flip]) : group_sum(ss, tpr);
        flip ^= 1;
        const float inv = inv_rms(tot, n, eps);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int vi = l + j * tpr;
            if (live && vi < nvec) {
                float o[VE];
#pragma unroll
                for (int e = 0; e < VE; ++e) o[e] = __fmul_rn(__fmul_rn(v[j][e], inv), gam[j][e]);
                st_stream(py + vi, Io<IO>::pack(o));
            }
        }
    }
}

// Any n, any alignment: one CTA per row, scalar accesses, the row read twice (the second pass hits cache).
// Thread t sums columns t, t + blockDim.x, ... in order, then the fixed CTA tree.
template <typename IO, typename WT>
__global__ void __launch_bounds__(256)
k_add_rmsnorm_generic(const IO* x_in, const IO* add, IO* x_out, const WT* w, IO* y, int n, long long T, float eps) {
    __shared__ float part[2][32];
    int flip = 0;
    for (long long row = blockIdx.x; row < T; row += gridDim.x) {
        const size_t off = (size_t)row * (size_t)n;
        const IO* xi = x_in + off;
        const IO* ai = add ? add + off : nullptr;
        IO* xo = x_out + off;
        IO* yo = y + off;
        float ss = 0.0f;
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            float v = Io<IO>::load1(xi + c);
            if (ai) {
                v = __fadd_rn(v, Io<IO>::load1(ai + c));
                Io<IO>::store1(xo + c, v);
                v = Io<IO>::round_trip(v);
            }
            ss = fmaf(v, v, ss);
        }
        const float tot = cta_sum(ss, part[flip]);
        flip ^= 1;
        const float inv = inv_rms(tot, n, eps);
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            // with add, the value is re-read from x_out: this thread wrote it above
            const float v = ai ? Io<IO>::load1(xo + c) : Io<IO>::load1(xi + c);
            Io<IO>::store1(yo + c, __fmul_rn(__fmul_rn(v, inv), gamma1(w, c)));
        }
    }
}

}  // namespace b200

#endif  // B200_RMSNORM_CUH
