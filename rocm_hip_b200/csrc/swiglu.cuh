// swiglu.cuh -- out = SiLU(g) * u, the B200 kernels behind gpu_swiglu and its bf16 sibling. Math of the reference's
// swiglu kernel (src/gpu_ops.hip:103-114) in the order of its CPU reference (src/qwen_ops.h:47,
// tests/forward_verify.cpp:365): (g / (1 + exp(-g))) * u.
//
// A flat elementwise map over n = rows * width values (dense FFN rows or expert-grouped rows: the order of rows does
// not matter to it), 3 s bytes per value. Each thread moves UNROLL 16-byte vectors of g and of u per step so that
// enough loads are in flight to cover HBM latency; the grid is a whole number of waves of resident CTAs.
//
// fp32 rows use the accurate expf and an IEEE division (within ~2 ulp of the CPU reference). 16-bit rows use
// ex2.approx and rcp.approx: their ~1e-6 relative error is far inside half a bf16 ulp (2e-3), so the rounded result
// differs from the rounded reference only when the exact value sits on a rounding boundary, by one ulp. The
// non-flushing rcp keeps the tiny results of very negative gates instead of cutting them to zero.

#ifndef B200_SWIGLU_CUH
#define B200_SWIGLU_CUH

#include "common.cuh"

namespace b200 {

template <bool FAST>
__device__ __forceinline__ float silu_mul(float g, float u) {
    if constexpr (FAST) {
        float e, r;
        asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
        asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
        return __fmul_rn(__fmul_rn(g, r), u);
    } else {
        return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
    }
}

template <typename IO, bool FAST, int UNROLL>
__global__ void __launch_bounds__(256)
k_swiglu(const IO* g, const IO* u, IO* out, long long n) {
    constexpr int VE = Io<IO>::VE;
    const long long nvec = n / VE;
    const uint4* pg = reinterpret_cast<const uint4*>(g);
    const uint4* pu = reinterpret_cast<const uint4*>(u);
    uint4* po = reinterpret_cast<uint4*>(out);
    const long long step = (long long)gridDim.x * blockDim.x * UNROLL;
    for (long long base = (long long)blockIdx.x * blockDim.x * UNROLL + threadIdx.x; base < nvec; base += step) {
        uint4 rg[UNROLL], ru[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const long long i = base + (long long)k * blockDim.x;
            if (i < nvec) {
                rg[k] = ld_stream(pg + i);
                ru[k] = ld_stream(pu + i);
            }
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const long long i = base + (long long)k * blockDim.x;
            if (i < nvec) {
                float a[VE], b[VE], o[VE];
                Io<IO>::unpack(rg[k], a);
                Io<IO>::unpack(ru[k], b);
#pragma unroll
                for (int e = 0; e < VE; ++e) o[e] = silu_mul<FAST>(a[e], b[e]);
                st_stream(po + i, Io<IO>::pack(o));
            }
        }
    }
    // the n % VE values after the last whole vector
    if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * VE)) {
        const long long i = nvec * VE + threadIdx.x;
        Io<IO>::store1(out + i, silu_mul<FAST>(Io<IO>::load1(g + i), Io<IO>::load1(u + i)));
    }
}

// Any alignment: one value per thread and step
template <typename IO, bool FAST>
__global__ void __launch_bounds__(256)
k_swiglu_scalar(const IO* g, const IO* u, IO* out, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        Io<IO>::store1(out + i, silu_mul<FAST>(Io<IO>::load1(g + i), Io<IO>::load1(u + i)));
}

// Any alignment, and rows whose gate / up halves sit at a stride (the experts' fused [gate | up] rows): out row r of h
// values from gate + r * gate_stride and up + r * up_stride. One value per thread and step.
template <typename IO, bool FAST>
__global__ void __launch_bounds__(256)
k_swiglu_strided(const IO* gate, const IO* up, IO* out, long long rows, int h, long long gate_stride,
                 long long up_stride) {
    const long long total = rows * h;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / h;
        const int c = (int)(i - r * h);
        Io<IO>::store1(out + i, silu_mul<FAST>(Io<IO>::load1(gate + r * gate_stride + c), Io<IO>::load1(up + r * up_stride + c)));
    }
}

// The strided form with 16-byte vectors: h, both strides and all three bases multiples of a vector
template <typename IO, bool FAST>
__global__ void __launch_bounds__(256)
k_swiglu_strided_vec(const IO* gate, const IO* up, IO* out, long long rows, int h, long long gate_stride,
                     long long up_stride) {
    constexpr int VE = Io<IO>::VE;
    const int hv = h / VE;
    const long long total = rows * hv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / hv;
        const int c = (int)(i - r * hv) * VE;
        const uint4 rg = ld_stream(gate + r * gate_stride + c);
        const uint4 ru = ld_stream(up + r * up_stride + c);
        float a[VE], b[VE], o[VE];
        Io<IO>::unpack(rg, a);
        Io<IO>::unpack(ru, b);
#pragma unroll
        for (int e = 0; e < VE; ++e) o[e] = silu_mul<FAST>(a[e], b[e]);
        st_stream(out + r * (long long)h + c, Io<IO>::pack(o));
    }
}

}  // namespace b200

#endif  // B200_SWIGLU_CUH
