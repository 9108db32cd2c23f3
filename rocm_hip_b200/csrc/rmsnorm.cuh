// rmsnorm.cuh -- residual add + RMSNorm over rows, the B200 kernels behind gpu_add_rmsnorm and its bf16 / fp16
// siblings. Math of the reference's add_rmsnorm / add_rmsnorm_rows (src/gpu_ops.hip:24-101) with the accumulation of
// its CPU reference (src/qwen_ops.cpp:8-13):
//   v = x_in + add (when add is set; v is stored to x_out); ss = sum of v^2 in double; inv = (float)(1 / sqrt(ss / n + eps));
//   y = (v * inv) * w, two fp32 multiplies left to right.
// The double sum costs nothing on a bandwidth-bound kernel and makes inv, hence y, the CPU reference's to the bit
// except when a double lands within an ulp of a float rounding boundary. For 16-bit rows the arithmetic is fp32 /
// double and the norm is taken of the value as stored in x_out (rounded), so a fused call gives the bits of a
// separate add followed by a norm.
//
// Layout: rows [T][n] contiguous. A row is read exactly once with 16-byte loads, VPT vectors per thread, kept packed
// in registers (so that many loads are in flight per thread at little register cost), reduced, scaled and written
// with 16-byte stores: 2 n s bytes per row without add, 4 n s with (s = bytes per value), the algorithmic minimum.
// Three kernels:
//   * k_add_rmsnorm_fast: the model-norm shapes (one CTA per row, the row exactly tpr * VPT vectors, fp32 or bf16,
//     gammas given): gammas in registers, packed fp32 math;
//   * k_add_rmsnorm: every other vectorisable shape: a lane group of tpr <= 32 threads per row (several rows per
//     CTA, shuffles only) or one CTA per row; gammas re-read per row through the read-only path;
//   * k_add_rmsnorm_generic: any width and alignment, scalar accesses.
// The launcher picks kernel, tpr and VPT from n and the storage type alone, never from T or the grid, so the
// summation order of a row is fixed. CTAs walk rows with a grid stride.

#ifndef B200_RMSNORM_CUH
#define B200_RMSNORM_CUH

#include "common.cuh"
#include "q8_side.cuh"

namespace b200 {

// CTA_ROW = false: lane groups of tpr threads (power of two <= 32), blockDim.x / tpr rows per pass.
// CTA_ROW = true : the whole CTA (tpr == blockDim.x) works on one row per pass.
template <typename IO, typename WT, int VPT, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 1024 : 256)
k_add_rmsnorm(const IO* x_in, const IO* add, IO* x_out, const WT* w, IO* y, int n, long long T, float eps, int tpr) {
    pdl_entry();
    constexpr int VE = Io<IO>::VE;
    __shared__ double part[2][32];
    const int nvec = n / VE;
    const int l = CTA_ROW ? (int)threadIdx.x : (int)threadIdx.x % tpr;
    const int g = CTA_ROW ? 0 : (int)threadIdx.x / tpr;
    const int rows_per_pass = CTA_ROW ? 1 : (int)blockDim.x / tpr;

    const double inv_n = 1.0 / (double)n;
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
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int vi = l + j * tpr;
            if (live && vi < nvec) {
                float v[VE];
                Io<IO>::unpack(rx[j], v);
                if (pa) {
                    float a[VE];
                    Io<IO>::unpack(ra[j], a);
#pragma unroll
                    for (int e = 0; e < VE; ++e) v[e] = __fadd_rn(v[e], a[e]);
                    rx[j] = Io<IO>::pack(v);              // the value as stored: the norm is taken of it
                    st_stream(po + vi, rx[j]);
                    if (sizeof(IO) < 4) Io<IO>::unpack(rx[j], v);
                }
#pragma unroll
                for (int e = 0; e < VE; ++e) ss = fma((double)v[e], (double)v[e], ss);
            }
        }
        const double tot = CTA_ROW ? cta_sum(ss, part[flip]) : group_sum(ss, tpr);
        flip ^= 1;
        const float inv = inv_rms(tot, inv_n, eps);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int vi = l + j * tpr;
            if (live && vi < nvec) {
                float v[VE], gam[VE];
                Io<IO>::unpack(rx[j], v);
                load_gamma<VE, WT>(w, vi * VE, gam);
#pragma unroll
                for (int e = 0; e < VE; ++e) v[e] = __fmul_rn(__fmul_rn(v[e], inv), gam[e]);
                st_stream(py + vi, Io<IO>::pack(v));
            }
        }
    }
}

// The common case, trimmed to the fewest instructions (these kernels are limited by instruction issue before HBM):
// one CTA per row, the row exactly tpr * VPT vectors (no masking anywhere), gammas present, fp32 or bf16 rows.
// Values travel as packed fp32 pairs: the add, the two multiplies and the bf16 packing are two-wide instructions,
// each lane rounded as the scalar instruction would. Same summation order as k_add_rmsnorm is NOT promised: a row
// width always maps to the same kernel, so a row's bits are still a function of the row alone.
// MAXT: largest CTA the instance is launched with (160, 320 or 512 threads); CTAs of up to 160 threads are held to 96
// registers so that four fit an SM (narrow rows of two vectors per thread to 48 / 80 so that eight / five do: a row of
// theirs is only 5 KB in flight), those of up to 320 to 102 so that two do.
// XH (fp32 rows only): y is also written rounded to bf16 (xh_bf16) or fp16 into xh, the 16-bit side copy the
// reference's producers write for their matmul consumers (src/q8_device.h:37-43,58): 2 more bytes per value written
// instead of a second kernel that reads y again.
// Q8 (fp32 rows, n % 256 == 0): y is also quantised into the Q8_0 and Q8_K activation formats from the registers that
// hold it, as the reference's producers do (src/q8_device.h:54-104, called at src/gpu_ops.hip:55,98): a Q8_0 block is
// 8 neighbouring lanes of one of the thread's vectors, a Q8_K block the 64 consecutive vectors of two 32-lane groups,
// whose keys meet in shared memory (one more CTA barrier per row). side: the xh pointer and the int8 outputs.
template <typename IO, int VPT, bool HAS_ADD, int MAXT, bool XH = false, bool Q8 = false>
__global__ void __launch_bounds__(MAXT, MAXT <= 160 ? (VPT <= 2 && !XH && !Q8 ? (HAS_ADD ? 5 : 8) : 4) : MAXT <= 320 ? (Q8 ? 3 : 2) : 1)
k_add_rmsnorm_fast(const IO* x_in, const IO* add, IO* x_out, const float* w, IO* y, int n, long long T, float eps,
                   const Q8Side side = Q8Side{}, int rows_per_cta = 0) {
    pdl_entry();
    static_assert(!(XH || Q8) || sizeof(IO) == 4, "the side outputs belong to fp32 rows");
    __shared__ Q8Half half_stat[Q8 ? 64 : 1];   // per 128 values of the row (n <= 8192)
    uint16_t* const xh = side.xh;
    const int xh_bf16 = side.xh_bf16;
    constexpr int NP = Io2<IO>::NP;
    // fp32 rows: every square goes into a double sum, which makes 1/rms, and with it y, the CPU reference's to the bit.
    // 16-bit rows: a thread's own 16 or 32 squares (each exact in fp32) are summed in two packed fp32 chains and only
    // the per-thread partials are combined in double. That saves a float-to-double conversion per value (the
    // conversion unit is the busiest pipe of the no-residual kernel: 93 % -> 97 % of the copy peak); 1/rms may then
    // differ from the reference's in its last bit, which moves a bf16 result only when it sits on a rounding tie.
    constexpr bool F32_PARTIAL = sizeof(IO) < 4;
    __shared__ double part[2][32];
    const int tpr = blockDim.x, l = threadIdx.x;
    const size_t row_vecs = (size_t)tpr * VPT;
    const double inv_n = 1.0 / (double)n;
    const uint4* px = reinterpret_cast<const uint4*>(x_in) + l;
    const uint4* pa = reinterpret_cast<const uint4*>(add) + l;
    uint4* po = reinterpret_cast<uint4*>(x_out) + l;
    uint4* py = reinterpret_cast<uint4*>(y) + l;
    // this thread's gammas stay in registers for all of the CTA's rows: re-reading them per row would put twice the
    // row's own bytes through L1 (fp32 gammas against 16-bit rows), and L1 throughput, not HBM, then sets the pace
    f2 gam[VPT][NP];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
#pragma unroll
        for (int h = 0; h < NP / 2; ++h) {
            const ulonglong2 g = __ldg(reinterpret_cast<const ulonglong2*>(w) + ((size_t)l + (size_t)j * tpr) * (NP / 2) + h);
            gam[j][2 * h] = g.x;
            gam[j][2 * h + 1] = g.y;
        }
    }
    // rows_per_cta > 0: CTA b takes the consecutive rows [b * rows_per_cta, (b + 1) * rows_per_cta) and retires (the grid
    // covers T); 0: the CTAs of a resident grid walk rows b, b + gridDim.x, ...
    const long long first = rows_per_cta ? (long long)blockIdx.x * rows_per_cta : (long long)blockIdx.x;
    const long long last = rows_per_cta ? (first + rows_per_cta < T ? first + rows_per_cta : T) : T;
    const long long rstride = rows_per_cta ? 1 : (long long)gridDim.x;
    size_t off = (size_t)first * row_vecs;
    const size_t step = (size_t)rstride * row_vecs;
    int flip = 0;
    // Where a thread holds few vectors (no residual, or narrow rows of two vectors per thread) the next row's loads
    // are issued before this row's reduction (two rows in flight per CTA); with the residual on rows of four vectors
    // per thread, x and add already double the bytes in flight and a second row would cost an SM its fourth CTA.
    constexpr bool PREFETCH = !HAS_ADD || VPT <= 2;
    uint4 rn[PREFETCH ? VPT : 1], rna[PREFETCH && HAS_ADD ? VPT : 1];
    if (PREFETCH && first < last) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            rn[j] = ld_stream(px + off + j * tpr);
            if (HAS_ADD) rna[j] = ld_stream(pa + off + j * tpr);
        }
    }
    for (long long row = first; row < last; row += rstride, off += step, flip ^= 1) {
        uint4 rx[VPT], ra[VPT];
        if (!PREFETCH) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                rx[j] = ld_stream(px + off + j * tpr);
                ra[j] = ld_stream(pa + off + j * tpr);
            }
        } else {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                rx[j] = rn[j];
                if (HAS_ADD) ra[j] = rna[j];
            }
            if (row + rstride < last) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    rn[j] = ld_stream(px + off + step + j * tpr);
                    if (HAS_ADD) rna[j] = ld_stream(pa + off + step + j * tpr);
                }
            }
        }
        double s0 = 0.0, s1 = 0.0;
        f2 sp = 0;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 v[NP];
            Io2<IO>::unpack(rx[j], v);
            if (HAS_ADD) {
                f2 a[NP];
                Io2<IO>::unpack(ra[j], a);
#pragma unroll
                for (int k = 0; k < NP; ++k) v[k] = add2(v[k], a[k]);
                rx[j] = Io2<IO>::pack(v);                    // the value as stored: the norm is taken of it
                st_stream(po + off + j * tpr, rx[j]);
                if (sizeof(IO) < 4) Io2<IO>::unpack(rx[j], v);
            }
            if (F32_PARTIAL) {
#pragma unroll
                for (int k = 0; k < NP; ++k) sp = fma2(v[k], v[k], sp);
            } else {
#pragma unroll
                for (int k = 0; k < NP; ++k) sumsq2(v[k], s0, s1);
            }
        }
        if (F32_PARTIAL) {
            float a, b;
            upk2(sp, a, b);
            s0 = (double)a;
            s1 = (double)b;
        }
        const double tot = cta_sum(s0 + s1, part[flip]);
        const float inv = inv_rms(tot, inv_n, eps);
        const f2 inv2 = pk2(inv, inv);
        float yq[Q8 ? VPT : 1][4];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            f2 v[NP];
            Io2<IO>::unpack(rx[j], v);
#pragma unroll
            for (int k = 0; k < NP; ++k) v[k] = mul2(mul2(v[k], inv2), gam[j][k]);
            st_stream(py + off + j * tpr, Io2<IO>::pack(v));
            if (XH) st_half4(xh + (off + j * tpr + l) * 4, v[0], v[NP > 1 ? 1 : 0], xh_bf16);
            if constexpr (Q8) {
                upk2(v[0], yq[j][0], yq[j][1]);
                upk2(v[1], yq[j][2], yq[j][3]);
            }
        }
        if constexpr (Q8) {
            unsigned qi[VPT];
            bool live[VPT], first[VPT];
            Q8Half blk[VPT];
            Q8Half* cell[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                qi[j] = ((unsigned)off + j * tpr + l) * 4u;
                live[j] = true;
                first[j] = (((l + j * tpr) >> 5) & 1) == 0;
                cell[j] = &half_stat[(l + j * tpr) >> 5];
            }
            q8v_phase_a<VPT>(yq, qi, live, side, cell);
            __syncthreads();   // (the next row's writes to half_stat come after its row-sum barrier)
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int hb = (l + j * tpr) >> 5;
                blk[j] = q8v_combine(half_stat[hb & ~1], half_stat[hb | 1]);
            }
            q8v_phase_b<VPT>(yq, qi, live, side, blk, first);
        }
    }
}

// Any n, any alignment: one CTA per row, scalar accesses, the row read twice (the second pass hits cache).
// Thread t sums columns t, t + blockDim.x, ... in order, then the fixed CTA tree.
template <typename IO, typename WT>
__global__ void __launch_bounds__(256)
k_add_rmsnorm_generic(const IO* x_in, const IO* add, IO* x_out, const WT* w, IO* y, int n, long long T, float eps) {
    __shared__ double part[2][32];
    const double inv_n = 1.0 / (double)n;
    int flip = 0;
    for (long long row = blockIdx.x; row < T; row += gridDim.x) {
        const size_t off = (size_t)row * (size_t)n;
        const IO* xi = x_in + off;
        const IO* ai = add ? add + off : nullptr;
        IO* xo = x_out + off;
        IO* yo = y + off;
        double ss = 0.0;
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            float v = Io<IO>::load1(xi + c);
            if (ai) {
                v = __fadd_rn(v, Io<IO>::load1(ai + c));
                Io<IO>::store1(xo + c, v);
                v = Io<IO>::round_trip(v);
            }
            ss = fma((double)v, (double)v, ss);
        }
        const double tot = cta_sum(ss, part[flip]);
        flip ^= 1;
        const float inv = inv_rms(tot, inv_n, eps);
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            // with add, the value is re-read from x_out: this thread wrote it above
            const float v = ai ? Io<IO>::load1(xo + c) : Io<IO>::load1(xi + c);
            Io<IO>::store1(yo + c, __fmul_rn(__fmul_rn(v, inv), gamma1(w, c)));
        }
    }
}

}  // namespace b200

#endif  // B200_RMSNORM_CUH
