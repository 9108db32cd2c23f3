// swiglu.cuh -- out = SiLU(g) * u, the B200 kernels behind gpu_swiglu and its bf16 sibling. Math of the reference's
// swiglu kernel (src/gpu_ops.hip:103-114) in the order of its CPU reference (src/qwen_ops.h:47,
// tests/forward_verify.cpp:365): (g / (1 + exp(-g))) * u.
//
// A flat elementwise map over n = rows * width values (dense FFN rows or expert-grouped rows: the order of rows does
// not matter to it), 3 s bytes per value. Each thread moves UNROLL 16-byte vectors of g and of u per step so that
// enough loads are in flight to cover HBM latency; CTAs walk tiles of 256 * UNROLL vectors with a grid stride.
//
// fp32 rows use the accurate expf and an IEEE division (within ~2 ulp of the CPU reference). 16-bit rows use
// ex2.approx and rcp.approx: their ~1e-6 relative error is far inside half a bf16 ulp (2e-3), so the rounded result
// differs from the rounded reference only when the exact value sits on a rounding boundary, by one ulp. The tiny
// results of very negative gates (below -87, where 1 + e exceeds 2^126 and its reciprocal is subnormal) are kept, not
// cut to zero, without the non-flushing reciprocal's range handling (six more instructions per value): the
// reciprocal is taken of (1 + e) / 16, which stays normal for every finite e, and the gate carries the 1 / 16
// (powers of two: the same mantissas, so the same bits wherever nothing is subnormal).

#ifndef B200_SWIGLU_CUH
#define B200_SWIGLU_CUH

#include "common.cuh"
#include "q8_side.cuh"

namespace b200 {

template <bool FAST>
__device__ __forceinline__ float silu_mul(float g, float u) {
    if constexpr (FAST) {
        float e, r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(g, -1.4426950408889634f)));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fmaf_rn(e, 0.0625f, 0.0625f)));   // 16 / (1 + e)
        return __fmul_rn(__fmul_rn(__fmul_rn(g, 0.0625f), r), u);
    } else {
        return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
    }
}

// SiLU(g) * u on packed pairs. FAST (16-bit rows): ex2.approx / rcp.approx, the scalings and products two-wide.
// ex2 flushes subnormal results to zero (they only occur for gates above 87, where 1 + e is 1 either way); the
// reciprocal's argument is scaled so that a gate below -87 still yields its tiny product instead of zero.
template <bool FAST>
__device__ __forceinline__ f2 silu_mul2(f2 g, f2 u) {
    float g0, g1;
    upk2(g, g0, g1);
    if constexpr (FAST) {
        float t0, t1, e0, e1, r0, r1;
        upk2(mul2(g, pk2(-1.4426950408889634f, -1.4426950408889634f)), t0, t1);
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(t0));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(t1));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(__fmaf_rn(e0, 0.0625f, 0.0625f)));   // 16 / (1 + e)
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(__fmaf_rn(e1, 0.0625f, 0.0625f)));
        return mul2(mul2(mul2(g, pk2(0.0625f, 0.0625f)), pk2(r0, r1)), u);
    } else {
        float u0, u1;
        upk2(u, u0, u1);
        return pk2(silu_mul<false>(g0, u0), silu_mul<false>(g1, u1));
    }
}

// Each CTA walks tiles of 256 * UNROLL vectors; inside a tile a thread's vectors are at tile + k * 256 + tid, so the
// per-access index arithmetic is 32-bit and only the tile base is 64-bit. All UNROLL loads of g and of u are issued
// before the first use. XH (fp32 rows, n a multiple of 4): out is also written rounded to bf16 (xh_bf16) or fp16 into
// xh, the 16-bit side copy of the reference's producers (src/q8_device.h:37-43,58).
template <typename IO, bool FAST, int UNROLL, bool XH = false>
__global__ void __launch_bounds__(256)
k_swiglu(const IO* g, const IO* u, IO* out, long long n, uint16_t* xh = nullptr, int xh_bf16 = 0) {
    pdl_entry();
    static_assert(!XH || sizeof(IO) == 4, "the 16-bit side copy belongs to fp32 rows");
    constexpr int VE = Io<IO>::VE, NP = VE / 2;
    const long long nvec = n / VE;
    constexpr int TILE = 256 * UNROLL;
    const long long ntiles = (nvec + TILE - 1) / TILE;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long v0 = tile * TILE;
        const uint4* pg = reinterpret_cast<const uint4*>(g) + v0 + threadIdx.x;
        const uint4* pu = reinterpret_cast<const uint4*>(u) + v0 + threadIdx.x;
        uint4* po = reinterpret_cast<uint4*>(out) + v0 + threadIdx.x;
        const int left = (int)(nvec - v0 < TILE ? nvec - v0 : TILE) - (int)threadIdx.x;  // vectors from this thread's first
        uint4 rg[UNROLL], ru[UNROLL];
        if (left > (UNROLL - 1) * 256) {   // whole tile for this thread: no per-access checks
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                rg[k] = ld_stream(pg + k * 256);
                ru[k] = ld_stream(pu + k * 256);
            }
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                f2 a[NP], b[NP];
                Io2<IO>::unpack(rg[k], a);
                Io2<IO>::unpack(ru[k], b);
#pragma unroll
                for (int e = 0; e < NP; ++e) a[e] = silu_mul2<FAST>(a[e], b[e]);
                st_stream(po + k * 256, Io2<IO>::pack(a));
                if (XH) st_half4(xh + (v0 + threadIdx.x + k * 256) * 4, a[0], a[NP > 1 ? 1 : 0], xh_bf16);
            }
        } else {
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                if (k * 256 < left) {
                    f2 a[NP], b[NP];
                    Io2<IO>::unpack(ld_stream(pg + k * 256), a);
                    Io2<IO>::unpack(ld_stream(pu + k * 256), b);
#pragma unroll
                    for (int e = 0; e < NP; ++e) a[e] = silu_mul2<FAST>(a[e], b[e]);
                    st_stream(po + k * 256, Io2<IO>::pack(a));
                    if (XH) st_half4(xh + (v0 + threadIdx.x + k * 256) * 4, a[0], a[NP > 1 ? 1 : 0], xh_bf16);
                }
            }
        }
    }
    // the n % VE values after the last whole vector
    if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * VE)) {
        const long long i = nvec * VE + threadIdx.x;
        Io<IO>::store1(out + i, silu_mul<FAST>(Io<IO>::load1(g + i), Io<IO>::load1(u + i)));
    }
}

// fp32 SwiGLU that also quantises its output into the Q8_0 and Q8_K activation formats (and the 16-bit copy when XH)
// from the registers that hold it, as the reference's swiglu does (src/gpu_ops.hip:113, src/q8_device.h:54-104): the
// tile walk of k_swiglu, in which the 256 threads' k-th vectors are 1024 consecutive values = four Q8_K blocks of two
// warps each; the two warps' keys meet in shared memory (one CTA barrier per tile; the key buffers alternate between
// tiles, so a tile's writes never meet the previous tile's reads). n % 32 == 0: a last partial Q8_K block gets its Q8_0
// blocks and an incomplete Q8_K part, as in the reference.
template <int UNROLL, bool XH>
__global__ void __launch_bounds__(256)
k_swiglu_q8(const float* g, const float* u, float* out, long long n, const Q8Side side) {
    pdl_entry();
    __shared__ Q8Half half_stat[2][UNROLL][8];
    const long long nvec = n / 4;
    constexpr int TILE = 256 * UNROLL;
    const long long ntiles = (nvec + TILE - 1) / TILE;
    const int warp = threadIdx.x >> 5;
    int flip = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, flip ^= 1) {
        const long long v0 = tile * TILE;
        const uint4* pg = reinterpret_cast<const uint4*>(g) + v0 + threadIdx.x;
        const uint4* pu = reinterpret_cast<const uint4*>(u) + v0 + threadIdx.x;
        uint4* po = reinterpret_cast<uint4*>(out) + v0 + threadIdx.x;
        const int left = (int)(nvec - v0 < TILE ? nvec - v0 : TILE) - (int)threadIdx.x;  // vectors from this thread's first
        uint4 rg[UNROLL], ru[UNROLL];
        bool live[UNROLL], first[UNROLL];
        unsigned qi[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            live[k] = k * 256 < left;
            first[k] = (warp & 1) == 0;
            qi[k] = ((unsigned)v0 + threadIdx.x + k * 256) * 4u;
            rg[k] = live[k] ? ld_stream(pg + k * 256) : make_uint4(0, 0, 0, 0);
            ru[k] = live[k] ? ld_stream(pu + k * 256) : make_uint4(0, 0, 0, 0);
        }
        float y[UNROLL][4];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            f2 a[2], b[2];
            Io2<float>::unpack(rg[k], a);
            Io2<float>::unpack(ru[k], b);
            a[0] = silu_mul2<false>(a[0], b[0]);
            a[1] = silu_mul2<false>(a[1], b[1]);
            if (live[k]) {
                st_stream(po + k * 256, Io2<float>::pack(a));
                if (XH) st_half4(side.xh + qi[k], a[0], a[1], side.xh_bf16);
            }
            upk2(a[0], y[k][0], y[k][1]);
            upk2(a[1], y[k][2], y[k][3]);
        }
        Q8Half blk[UNROLL];
        Q8Half* cell[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) cell[k] = &half_stat[flip][k][warp];
        q8v_phase_a<UNROLL>(y, qi, live, side, cell);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) blk[k] = q8v_combine(half_stat[flip][k][warp & ~1], half_stat[flip][k][warp | 1]);
        q8v_phase_b<UNROLL>(y, qi, live, side, blk, first);
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
