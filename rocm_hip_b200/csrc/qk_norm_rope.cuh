// qk_norm_rope.cuh -- per-head q/k RMSNorm fused with NeoX rotary embedding, the B200 kernels behind
// gpu_qk_norm_rope. Math of the reference's norm_rope<D> (src/attention.hip:212-236) as its CPU references state it
// (qwen_rmsnorm + qwen_rope_neox, src/qwen_ops.cpp:8-24; qk_ref, tests/forward_verify.cpp:835-853): per head
//   x *= rsqrt(mean(x^2) + eps) * w[d];  pairs (i, i + n_rot/2), i < rot_pairs, rotate by theta_i = pos * base^(-2i/n_rot)
//   (divided by ff[i] when frequency factors are given); dims >= n_rot and pairs >= rot_pairs stay as they are.
// Unlike the reference kernel, which forms theta in fp32 (tested to 1e-3 at position 2499), the angle here is the
// double product pos * inv_freq[i] with inv_freq built on the host by the CPU reference's own expression, and
// cos / sin are evaluated in double and rounded once: that is what holds 1e-5 at positions in the hundreds of thousands.
//
// A CTA pass handles a tile of consecutive tokens (4 in long batches): all of their n_q + n_kv heads. A head of D
// values is NV = D / VE 16-byte vectors, owned by NV / (2 PPT) threads. Each thread owns PPT pairs of vectors; a
// rotating thread owns the vector of a rotation pair's low half and the vector of its high half, so the rotation
// needs no exchange, the row is read once and written once (2 D s bytes per head), and the sum of squares is a
// shuffle reduction inside the head's lanes. A tile's cos / sin (n_rot / 2 each per token) sit in shared memory,
// shared by all heads: computed there once, in double, or (table route) copied there from the tables k_rope_table
// filled once for the whole forward pass.
// Four kernels: k_qk_norm_rope_fast (long batches of the usual shapes: everything static, gammas and tables in
// bank-conflict-free shared-memory layouts; TAB: the next tile's tables fetched by cp.async one pass ahead, else
// computed at the end of a pass with its own sincos); k_qk_norm_rope (any vectorisable shape, any batch length,
// frequency factors); k_qk_norm_rope_generic (any head size and alignment, scalar); k_rope_table.

#ifndef B200_QK_NORM_ROPE_CUH
#define B200_QK_NORM_ROPE_CUH

#include "common.cuh"
#include "kv_store.cuh"

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
    // KVC kernels only: the K heads go, rounded to fp16, into the block-major KV cache instead of k_out
    // (the K write of the reference's attn_prep, src/attention.hip:286-299; row addressing :38-42)
    __half* k_cache;
    int kv_stride, kv_shift;
    long long kv_bstride;
    // cos / sin of every token's angles computed beforehand (k_rope_table): [T][n_rot / 2] fp32 each, row t = token t,
    // (1, 0) in the pairs that do not rotate. NULL: the kernel evaluates them itself.
    const float* cos_tab;
    const float* sin_tab;
};

// VE consecutive values of token t's K row, starting at element e of the row (e a multiple of VE), into the cache
template <int VE>
__device__ __forceinline__ void kv_put(const QkArgs& a, long long t, int e, const float* v) {
    const int pos = a.positions ? a.positions[t] : a.pos0 + (int)t;
    __half* row = a.k_cache + kv_row(pos, a.kv_stride, a.kv_shift, a.kv_bstride) + e;
    if constexpr (VE == 8) {
        st_stream(row, Io<__half>::pack(v));
    } else {
        const uint2 r = make_uint2(pack_f16(v[0], v[1]), pack_f16(v[2], v[3]));
        asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(row), "r"(r.x), "r"(r.y) : "memory");
    }
}

// Rotates two pairs at once: (x0, x1) -> (x0 c - x1 s, x0 s + x1 c) with every product and sum rounded separately, as
// the CPU reference evaluates it (src/qwen_ops.cpp:21-22). The four products are two-wide multiplies; the sums are
// scalar add.rn / sub.rn because the assembler contracts a two-wide multiply that feeds a two-wide add into a fused
// multiply-add even when both carry .rn (measured: 26 % of results differ in the last bit), which it never does to
// the scalar forms. (Writing the sums as fused multiply-adds by an opaque +1 / -1, which nothing can contract, gives the
// same bits with fewer instructions, but measured 3 % slower in the table-reading tile kernel.)
__device__ __forceinline__ void rotate2(f2 x0, f2 x1, f2 c, f2 s, float* lo, float* hi) {
    float a0, a1, b0, b1, c0, c1, d0, d1;
    upk2(mul2(x0, c), a0, a1);
    upk2(mul2(x1, s), b0, b1);
    upk2(mul2(x0, s), c0, c1);
    upk2(mul2(x1, c), d0, d1);
    lo[0] = __fsub_rn(a0, b0);
    lo[1] = __fsub_rn(a1, b1);
    hi[0] = __fadd_rn(c0, d0);
    hi[1] = __fadd_rn(c1, d1);
}

// cos / sin of the angles of `nt` consecutive tokens starting at t0, spread over all threads of the CTA:
// cos_t / sin_t [token][n_rot / 2]. Pairs at or beyond rot_pairs get (1, 0): x0 * 1 - x1 * 0 is x0 to the bit, so the
// rotation loop needs no per-pair test.
//
// chunk_lanes > 0 selects the layout the trimmed kernel reads without shared-memory bank conflicts: a lane owns VE
// consecutive pairs and fetches them as 16-byte chunks of 4, so chunk c of lane l is stored at ((c * chunk_lanes + l) * 4)
// within the token's row: the 8 lanes of a quarter-warp then read 128 contiguous bytes (natural order puts them 32
// bytes apart, two lanes per bank). chunk_lanes = number of rotating lanes per head; ve = pairs per lane.
// sin and cos of a double-precision angle, 0 <= |x| < 2^32 * pi/2 (every int32 position times a multiplier <= 1), without
// the library routine's large-argument path (whose local array and register needs weigh on the whole kernel):
// k = rint(x * 2/pi); r = x - k * pi/2 with pi/2 split into three 21-bit pieces and a tail, so every k * piece product
// is exact for |k| < 2^32 (Cody-Waite); then the classic degree-13 / degree-14 minimax polynomials on [-pi/4, pi/4]
// (the coefficients of fdlibm's __kernel_sin / __kernel_cos), each below one ulp. Rounded to float the results are
// those of the CPU reference's libm except when the exact value lies within ~2 double ulps of a float rounding tie.
__device__ __forceinline__ void sincos_cw(double x, double* sn, double* cs) {
    const double k = rint(x * 0.6366197723675814);
    double r = fma(-k, 1.570796012878418, x);          // 0x1.921fb00000000p+0
    r = fma(-k, 3.139164164167596e-07, r);             // 0x1.5110b00000000p-22
    r = fma(-k, 6.22337468017542e-14, r);              // 0x1.1846a00000000p-44
    r = fma(-k, -2.508278806334166e-20, r);            // tail of pi/2
    const double z = r * r;
    double ps = fma(z, 1.58969099521155010221e-10, -2.50507602534068634195e-08);
    ps = fma(z, ps, 2.75573137070700676789e-06);
    ps = fma(z, ps, -1.98412698298579493134e-04);
    ps = fma(z, ps, 8.33333333332248946124e-03);
    ps = fma(z, ps, -1.66666666666666324348e-01);
    const double s = fma(z * r, ps, r);
    double pc = fma(z, -1.13596475577881948265e-11, 2.08757232129817482790e-09);
    pc = fma(z, pc, -2.75573143513906633035e-07);
    pc = fma(z, pc, 2.48015872894767294178e-05);
    pc = fma(z, pc, -1.38888888888741095749e-03);
    pc = fma(z, pc, 4.16666666666666019037e-02);
    const double c = 1.0 - fma(-(z * z), pc, 0.5 * z);
    const int q = (int)((long long)k & 3);
    *sn = (q & 1) ? c : s;
    *cs = (q & 1) ? s : c;
    if (q == 1 || q == 2) *cs = -*cs;
    if (q >= 2) *sn = -*sn;
}

// inv_freq: the angle multipliers in SHARED memory. (Indexing the kernel-parameter copy with a per-thread index makes
// the 32 lanes' constant-bank reads serialise: measured 0.15 of this kernel's time.)
template <bool FAST_TRIG = false>
__device__ __forceinline__ void tokens_cos_sin(float* cos_t, float* sin_t, const QkArgs& a, const double* inv_freq,
                                               long long t0, int nt, int chunk_lanes = 0, int ve = 4) {
    const int half = a.n_rot >> 1, total = nt * half;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int tt = idx / half, i = idx - tt * half;
        float c = 1.0f, s = 0.0f;
        if (!FAST_TRIG && a.cos_tab) {   // uniform: the tables were computed beforehand
            c = __ldg(a.cos_tab + (size_t)(t0 + tt) * half + i);
            s = __ldg(a.sin_tab + (size_t)(t0 + tt) * half + i);
        } else if (i < a.rot_pairs) {
            const int pos = a.positions ? a.positions[t0 + tt] : a.pos0 + (int)(t0 + tt);
            double theta = (double)pos * inv_freq[i];
            if (a.ff) theta /= (double)a.ff[i];
            double ds, dc;
            if (FAST_TRIG) sincos_cw(theta, &ds, &dc);   // (the launcher guarantees |theta| < 2^31 here)
            else sincos(theta, &ds, &dc);
            c = (float)dc;
            s = (float)ds;
        }
        int at = idx;
        if (chunk_lanes > 0) {
            const int l = i / ve, r = i - l * ve;
            at = tt * half + (((r >> 2) * chunk_lanes + l) << 2) + (r & 3);
        }
        cos_t[at] = c;
        sin_t[at] = s;
    }
}

// The cos / sin rows of `nt` consecutive tokens starting at t0, from the tables in global memory into the
// chunk-major shared-memory layout of tokens_cos_sin (chunk c of lane l at ((c * chunk_lanes + l) * 4) within the
// token's row), as 16-byte asynchronous copies spread over the CTA. n_rot / 2 a multiple of 4, tables 16-byte aligned.
__device__ __forceinline__ void tile_tables_async(float* cos_t, float* sin_t, const QkArgs& a, long long t0, int nt,
                                                  int chunk_lanes, int ve, int half) {
    const int cpr = half >> 2, C = ve >> 2;   // chunks per token row, chunks per lane
    const float* gc = a.cos_tab + (size_t)t0 * half;
    const float* gs = a.sin_tab + (size_t)t0 * half;
    for (int idx = threadIdx.x; idx < 2 * nt * cpr; idx += blockDim.x) {
        const int which = idx >= nt * cpr, r = idx - which * nt * cpr;
        const int tt = r / cpr, ch = r - tt * cpr;
        const int l = ch / C, c = ch - l * C;
        const int at = tt * half + ((c * chunk_lanes + l) << 2);
        cp_async16((which ? sin_t : cos_t) + at, (which ? gs : gc) + (size_t)r * 4);
    }
}

// Copies the n_rot / 2 angle multipliers from the kernel parameters into shared memory (thread i reads entry i of the
// parameter block: done once per CTA) and synchronises the CTA.
__device__ __forceinline__ void stage_inv_freq(double* dst, const RopeFreq& fr, int half) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) dst[i] = fr.inv_freq[i];
    __syncthreads();
}

// PPT: pairs of vectors per thread. Threads per head tph = D / VE / (2 PPT), a power of two <= 32.
// TT: tokens per CTA pass. All of a pass's loads are issued before its cos / sin are computed, so TT * 2 PPT 16-byte
// loads per thread are in flight while the double-precision sincos runs; the tables of the pass are shared by all heads.
// Dynamic shared memory: 2 passes x (cos, sin) x TT x n_rot / 2 floats (a pass writes one half while slower threads
// may still read the other). Values travel as packed fp32 pairs (two-wide multiplies, adds and subtractions, each lane
// rounded as the scalar instruction would).
template <typename IO, int PPT, int TT, bool KVC = false>
__global__ void __launch_bounds__(384, 2)
k_qk_norm_rope(const QkArgs a, const __grid_constant__ RopeFreq fr) {
    pdl_entry();
    constexpr int VE = Io<IO>::VE, NP = VE / 2;
    extern __shared__ __align__(16) float tab_all[];
    __shared__ double invf[B200_MAX_ROT_PAIRS];
    stage_inv_freq(invf, fr, a.n_rot >> 1);
    const int D = a.D, NV = D / VE, tph = NV / (2 * PPT);
    const int R = a.n_rot / VE;      // vectors in the rotary part
    const int P = R / 2;             // pairs of vectors (low half, high half)
    const int half = a.n_rot >> 1;
    const int heads = a.n_q + a.n_kv;
    const int heads_per_pass = blockDim.x / tph;
    const int l = threadIdx.x % tph, hslot = threadIdx.x / tph;
    const double inv_n = 1.0 / (double)D;

    // this thread's vector slots within a head: slot s < P pairs vector s with s + P (a rotation pair's two halves);
    // the vectors past the rotary part are split the same way, first half / second half, so that the lanes of a head
    // always touch consecutive vectors
    int vlo[PPT], vhi[PPT];
    bool rot[PPT];
    const int Q = (NV - R) / 2;
#pragma unroll
    for (int p = 0; p < PPT; ++p) {
        const int s = l + p * tph;  // 0 .. NV/2-1
        rot[p] = s < P;
        vlo[p] = rot[p] ? s : R + (s - P);
        vhi[p] = rot[p] ? s + P : R + (s - P) + Q;
    }

    int flip = 0;
    const long long ntiles = (a.T + TT - 1) / TT;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, flip ^= 1) {
        const long long t0 = tile * TT;
        const int nt = (int)(a.T - t0 < TT ? a.T - t0 : TT);
        float* cos_t = tab_all + (size_t)flip * 2 * TT * half;
        float* sin_t = cos_t + TT * half;
        bool tables_done = false;
        for (int h0 = 0; h0 < heads; h0 += heads_per_pass) {
            const int h = h0 + hslot;
            const bool live = h < heads;
            const bool isq = h < a.n_q;
            const float* gamma = isq ? a.q_norm : a.k_norm;
            const size_t in_tok = isq ? (size_t)a.n_q * a.q_stride : (size_t)a.n_kv * D;   // values per token row
            const size_t out_tok = isq ? (size_t)a.n_q * D : (size_t)a.n_kv * D;
            const uint4* src = reinterpret_cast<const uint4*>(
                isq ? static_cast<const IO*>(a.qfull) + (size_t)t0 * in_tok + (size_t)h * a.q_stride
                    : static_cast<const IO*>(a.k) + (size_t)t0 * in_tok + (size_t)(h - a.n_q) * D);
            uint4* dst = reinterpret_cast<uint4*>(
                isq ? static_cast<IO*>(a.q_out) + (size_t)t0 * out_tok + (size_t)h * D
                    : static_cast<IO*>(a.k_out) + (size_t)t0 * out_tok + (size_t)(h - a.n_q) * D);
            const unsigned in_vec = (unsigned)(in_tok / VE), out_vec = (unsigned)(out_tok / VE);  // vectors per token
            uint4 rlo[TT][PPT], rhi[TT][PPT];
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                if (live && tt < nt) {
#pragma unroll
                    for (int p = 0; p < PPT; ++p) {
                        rlo[tt][p] = ld_stream(src + (tt * in_vec + (unsigned)vlo[p]));
                        rhi[tt][p] = ld_stream(src + (tt * in_vec + (unsigned)vhi[p]));
                    }
                }
            }
            if (!tables_done) {  // uniform over the CTA
                tokens_cos_sin(cos_t, sin_t, a, invf, t0, nt, P, VE);   // lane-contiguous chunks (no bank conflicts)
                __syncthreads();
                tables_done = true;
            }
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                if (tt >= nt) break;  // uniform
                f2 lo[PPT][NP], hi[PPT][NP];
                double s0 = 0.0, s1 = 0.0;
                if (live) {
#pragma unroll
                    for (int p = 0; p < PPT; ++p) {
                        Io2<IO>::unpack(rlo[tt][p], lo[p]);
                        Io2<IO>::unpack(rhi[tt][p], hi[p]);
                        if (a.do_norm) {
#pragma unroll
                            for (int k = 0; k < NP; ++k) sumsq2(lo[p][k], s0, s1);
#pragma unroll
                            for (int k = 0; k < NP; ++k) sumsq2(hi[p][k], s0, s1);
                        }
                    }
                }
                if (a.do_norm) {  // uniform
                    const float inv = inv_rms(group_sum(s0 + s1, tph), inv_n, a.eps);
                    const f2 inv2 = pk2(inv, inv);
                    if (live) {
#pragma unroll
                        for (int p = 0; p < PPT; ++p) {
#pragma unroll
                            for (int k = 0; k < NP; k += 2) {
                                // (the launcher substitutes a vector of ones for a missing gamma)
                                const ulonglong2 gl = __ldg(reinterpret_cast<const ulonglong2*>(gamma + vlo[p] * VE) + (k >> 1));
                                const ulonglong2 gh = __ldg(reinterpret_cast<const ulonglong2*>(gamma + vhi[p] * VE) + (k >> 1));
                                lo[p][k] = mul2(mul2(lo[p][k], inv2), gl.x);
                                hi[p][k] = mul2(mul2(hi[p][k], inv2), gh.x);
                                if (k + 1 < NP) {
                                    lo[p][k + 1] = mul2(mul2(lo[p][k + 1], inv2), gl.y);
                                    hi[p][k + 1] = mul2(mul2(hi[p][k + 1], inv2), gh.y);
                                }
                            }
                        }
                    }
                }
                if (live) {
#pragma unroll
                    for (int p = 0; p < PPT; ++p) {
                        float flo[VE], fhi[VE];
                        if (rot[p]) {
                            // pairs vlo * VE .. + VE - 1 of this token's tables
                            // chunk c of rotating slot vlo: [(c * P + vlo) * 4] within the token's row
                            const ulonglong2* ct = reinterpret_cast<const ulonglong2*>(cos_t + tt * half) + vlo[p];
                            const ulonglong2* st = reinterpret_cast<const ulonglong2*>(sin_t + tt * half) + vlo[p];
#pragma unroll
                            for (int k = 0; k < NP; k += 2) {
                                const ulonglong2 c = ct[(k >> 1) * P], sn = st[(k >> 1) * P];
                                rotate2(lo[p][k], hi[p][k], c.x, sn.x, flo + 2 * k, fhi + 2 * k);
                                rotate2(lo[p][k + 1], hi[p][k + 1], c.y, sn.y, flo + 2 * k + 2, fhi + 2 * k + 2);
                            }
                        } else {
#pragma unroll
                            for (int k = 0; k < NP; ++k) {
                                upk2(lo[p][k], flo[2 * k], flo[2 * k + 1]);
                                upk2(hi[p][k], fhi[2 * k], fhi[2 * k + 1]);
                            }
                        }
                        if (KVC && !isq) {
                            kv_put<VE>(a, t0 + tt, (h - a.n_q) * D + vlo[p] * VE, flo);
                            kv_put<VE>(a, t0 + tt, (h - a.n_q) * D + vhi[p] * VE, fhi);
                        } else {
                            st_stream(dst + (tt * out_vec + (unsigned)vlo[p]), Io<IO>::pack(flo));
                            st_stream(dst + (tt * out_vec + (unsigned)vhi[p]), Io<IO>::pack(fhi));
                        }
                    }
                }
            }
        }
    }
}

// The common case with everything that can be static made static: the CTA is exactly (heads x tph) threads (one head
// chunk, every thread live), T is a multiple of TT (the launcher gives the tail tokens to k_qk_norm_rope), PPT = 1,
// normalisation on. FULL: n_rot == D, so every thread rotates. The gammas of q and k sit in shared memory next to the
// tables (read with immediate offsets: no address arithmetic in the token loop).
// Shared memory: [2 * D floats: q gamma, k gamma][2 passes x (cos, sin) x TT x n_rot / 2 floats].
//
// TAB: the cos / sin of every token come from tables in global memory (a.cos_tab, a.sin_tab: k_rope_table fills them
// once per forward pass and every layer's call reads them). A tile's 2 * TT * n_rot / 2 floats are fetched into the
// same shared-memory layout with 16-byte cp.async copies issued one pass ahead, so no trigonometry and no double
// arithmetic beyond the sum of squares remains in the streaming kernel: it fits 3 to 5 CTAs per SM where the kernel
// that evaluates sin / cos itself fits 2. MINB: resident CTAs the register budget is held to.
// DS / NR: head size and rotary width fixed at compile time (0: taken from the arguments), which turns every
// shared-memory offset of the token loop into an immediate.
template <typename IO, int TT, bool FULL, bool KVC = false, bool TAB = false, int MINB = (TT <= 2 ? 3 : 2), int DS = 0,
          int NR = 0>
__global__ void __launch_bounds__(384, MINB)
k_qk_norm_rope_fast(const QkArgs a, const __grid_constant__ RopeFreq fr) {
    pdl_entry();
    constexpr int VE = Io<IO>::VE, NP = VE / 2;
    extern __shared__ __align__(16) float smem_all[];
    __shared__ double invf[TAB ? 1 : B200_MAX_ROT_PAIRS];
    const int n_rot = NR ? NR : a.n_rot;
    if (!TAB) stage_inv_freq(invf, fr, n_rot >> 1);
    const int D = DS ? DS : a.D, NV = D / VE, tph = NV / 2;
    const int R = n_rot / VE, P = R / 2, half = n_rot >> 1;
    const int l = threadIdx.x % tph, h = threadIdx.x / tph;
    const bool isq = h < a.n_q;
    const double inv_n = 1.0 / (double)D;
    float* gam_s = smem_all;
    float* tab = smem_all + 2 * D;
    constexpr int C = VE / 4;        // 16-byte chunks of 4 floats per vector's worth of gammas / pairs
    // gammas in shared memory as [q | k][low vector, high vector][chunk][lane][4]: the lanes of a head read
    // consecutive 16-byte chunks (no bank conflicts), each lane exactly the gammas of the two vectors it owns
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
        const int which = i / D, r = i - which * D;
        const int hv = r / (D / 2), r2 = r - hv * (D / 2);
        const int c = r2 / (tph * 4), r3 = r2 - c * (tph * 4);
        const int ll = r3 >> 2, j = r3 & 3;
        const bool lrot = FULL || ll < P;
        const int vec = hv == 0 ? (lrot ? ll : R + (ll - P)) : (lrot ? ll + P : R + (ll - P) + (NV - R) / 2);
        gam_s[i] = (which == 0 ? a.q_norm : a.k_norm)[vec * VE + 4 * c + j];
    }
    const bool rot = FULL || l < P;
    const int vlo = rot ? l : R + (l - P);
    const int vhi = rot ? l + P : R + (l - P) + (NV - R) / 2;
    // chunk c of the low vector's gammas at glo[c * tph], of the high vector's at ghi[c * tph]
    const ulonglong2* glo = reinterpret_cast<const ulonglong2*>(gam_s + (isq ? 0 : D)) + l;
    const ulonglong2* ghi = glo + C * tph;
    const int PL = FULL ? tph : P;   // rotating lanes per head
    // this thread's place in a token row, in 16-byte vectors
    const unsigned in_vec = (unsigned)((isq ? (size_t)a.n_q * a.q_stride : (size_t)a.n_kv * D) / VE);
    const unsigned out_vec = (unsigned)((isq ? (size_t)a.n_q * D : (size_t)a.n_kv * D) / VE);
    const unsigned in_head = (unsigned)((isq ? (size_t)h * a.q_stride : (size_t)(h - a.n_q) * D) / VE);
    const unsigned out_head = (unsigned)((isq ? h : h - a.n_q) * NV);
    const uint4* in_base = reinterpret_cast<const uint4*>(isq ? a.qfull : a.k) + in_head;
    uint4* out_base = reinterpret_cast<uint4*>(isq ? a.q_out : a.k_out) + out_head;
    __syncthreads();

    int flip = 0;
    const long long ntiles = a.T / TT, tile0 = blockIdx.x, tstride = gridDim.x;
    // The tables of a tile are computed at the END of the pass before it (the first tile's here), into the buffer the
    // pass before that used: the double-precision sincos then runs while none of a pass's loaded vectors are live, so
    // its registers do not compete with them (computing the tables between the loads and their use cost 15 %).
    if (tile0 < ntiles) {
        if (TAB) tile_tables_async(tab, tab + TT * half, a, tile0 * TT, TT, PL, VE, half);
        else tokens_cos_sin<true>(tab, tab + TT * half, a, invf, tile0 * TT, TT, PL, VE);
    }
    for (long long tile = tile0; tile < ntiles; tile += tstride, flip ^= 1) {
        const long long t0 = tile * TT;
        const uint4* src = in_base + (size_t)t0 * in_vec;
        uint4* dst = out_base + (size_t)t0 * out_vec;
        uint4 rlo[TT], rhi[TT];
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            rlo[tt] = ld_stream(src + (tt * in_vec + (unsigned)vlo));
            rhi[tt] = ld_stream(src + (tt * in_vec + (unsigned)vhi));
        }
        float* cos_t = tab + flip * (2 * TT * half);
        float* sin_t = cos_t + TT * half;
        if (TAB) cp_async_wait_all();   // this thread's copies of this tile's tables have landed
        __syncthreads();   // this tile's tables (written during the previous pass) are complete
        if (TAB && tile + tstride < ntiles) {   // the other buffer was last read one pass ago, before this barrier
            float* ncos = tab + (flip ^ 1) * (2 * TT * half);
            tile_tables_async(ncos, ncos + TT * half, a, (tile + tstride) * TT, TT, PL, VE, half);
        }
        const ulonglong2* ct = reinterpret_cast<const ulonglong2*>(cos_t) + l;   // chunk c of token tt: [(tt * half) / 4 + c * PL]
        const ulonglong2* st = reinterpret_cast<const ulonglong2*>(sin_t) + l;
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            f2 lo[NP], hi[NP];
            Io2<IO>::unpack(rlo[tt], lo);
            Io2<IO>::unpack(rhi[tt], hi);
            double s0 = 0.0, s1 = 0.0;
#pragma unroll
            for (int k = 0; k < NP; ++k) sumsq2(lo[k], s0, s1);
#pragma unroll
            for (int k = 0; k < NP; ++k) sumsq2(hi[k], s0, s1);
            const float inv = inv_rms(group_sum(s0 + s1, tph), inv_n, a.eps);
            const f2 inv2 = pk2(inv, inv);
#pragma unroll
            for (int k = 0; k < NP; k += 2) {
                const ulonglong2 gl = glo[(k >> 1) * tph], gh = ghi[(k >> 1) * tph];
                lo[k] = mul2(mul2(lo[k], inv2), gl.x);
                hi[k] = mul2(mul2(hi[k], inv2), gh.x);
                lo[k + 1] = mul2(mul2(lo[k + 1], inv2), gl.y);
                hi[k + 1] = mul2(mul2(hi[k + 1], inv2), gh.y);
            }
            float flo[VE], fhi[VE];
            if (rot) {
#pragma unroll
                for (int k = 0; k < NP; k += 2) {
                    const ulonglong2 c = ct[(tt * half) / 4 + (k >> 1) * PL], sn = st[(tt * half) / 4 + (k >> 1) * PL];
                    rotate2(lo[k], hi[k], c.x, sn.x, flo + 2 * k, fhi + 2 * k);
                    rotate2(lo[k + 1], hi[k + 1], c.y, sn.y, flo + 2 * k + 2, fhi + 2 * k + 2);
                }
            } else {
#pragma unroll
                for (int k = 0; k < NP; ++k) {
                    upk2(lo[k], flo[2 * k], flo[2 * k + 1]);
                    upk2(hi[k], fhi[2 * k], fhi[2 * k + 1]);
                }
            }
            if (KVC && !isq) {
                kv_put<VE>(a, t0 + tt, (h - a.n_q) * D + vlo * VE, flo);
                kv_put<VE>(a, t0 + tt, (h - a.n_q) * D + vhi * VE, fhi);
            } else {
                st_stream(dst + (tt * out_vec + (unsigned)vlo), Io<IO>::pack(flo));
                st_stream(dst + (tt * out_vec + (unsigned)vhi), Io<IO>::pack(fhi));
            }
        }
        if (!TAB && tile + tstride < ntiles) {   // the other buffer was last read one pass ago, before this pass's barrier
            float* ncos = tab + (flip ^ 1) * (2 * TT * half);
            tokens_cos_sin<true>(ncos, ncos + TT * half, a, invf, (tile + tstride) * TT, TT, PL, VE);
        }
    }
}

// Any head size, rotary width and alignment: one CTA pass per token, heads one after the other, the normalised head
// staged in shared memory so that a value can read its rotation partner (the reference kernel's own scheme).
// D <= 1024.
template <typename IO>
__global__ void __launch_bounds__(128)
k_qk_norm_rope_generic(const QkArgs a, const __grid_constant__ RopeFreq fr) {
    __shared__ float cos_t[B200_MAX_ROT_PAIRS], sin_t[B200_MAX_ROT_PAIRS];
    __shared__ double invf[B200_MAX_ROT_PAIRS];
    stage_inv_freq(invf, fr, a.n_rot >> 1);
    __shared__ float v[1024];
    __shared__ double part[2][32];
    const int D = a.D, half = a.n_rot / 2, heads = a.n_q + a.n_kv;
    const double inv_n = 1.0 / (double)a.D;
    int flip = 0;
    for (long long t = blockIdx.x; t < a.T; t += gridDim.x) {
        __syncthreads();  // the previous token's tables and head are no longer read
        tokens_cos_sin(cos_t, sin_t, a, invf, t, 1);
        for (int h = 0; h < heads; ++h) {
            const bool isq = h < a.n_q;
            const IO* src = isq ? static_cast<const IO*>(a.qfull) + ((size_t)t * a.n_q + h) * a.q_stride
                                : static_cast<const IO*>(a.k) + ((size_t)t * a.n_kv + (h - a.n_q)) * D;
            IO* dst = isq ? static_cast<IO*>(a.q_out) + ((size_t)t * a.n_q + h) * D
                          : static_cast<IO*>(a.k_out) + ((size_t)t * a.n_kv + (h - a.n_q)) * D;
            const float* gamma = isq ? a.q_norm : a.k_norm;
            double ss = 0.0;
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                const float x = Io<IO>::load1(src + d);
                v[d] = x;
                ss = fma((double)x, (double)x, ss);
            }
            float inv = 1.0f;
            if (a.do_norm) {
                inv = inv_rms(cta_sum(ss, part[flip]), inv_n, a.eps);
                flip ^= 1;
                for (int d = threadIdx.x; d < D; d += blockDim.x)  // this thread's own values
                    v[d] = __fmul_rn(__fmul_rn(v[d], inv), gamma1(gamma, d));
            }
            __syncthreads();
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                float x = v[d];
                const int i = d < half ? d : d - half;
                if (d < a.n_rot && i < a.rot_pairs) {
                    const float c = cos_t[i], sn = sin_t[i];
                    const float x0 = v[i], x1 = v[i + half];
                    x = d < half ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn))
                                 : __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
                }
                if (!isq && a.k_cache) {
                    const int pos = a.positions ? a.positions[t] : a.pos0 + (int)t;
                    a.k_cache[kv_row(pos, a.kv_stride, a.kv_shift, a.kv_bstride) + (size_t)(h - a.n_q) * D + d] = __float2half_rn(x);
                } else {
                    Io<IO>::store1(dst + d, x);
                }
            }
            __syncthreads();  // v is rewritten by the next head
        }
    }
}

// The cos / sin tables the TAB kernels read: cos_out / sin_out [T][half] fp32, row t = token t at positions[t] (or
// pos0 + t), entry i = cos / sin of pos * inv_freq[i] (/ ff[i]) formed and evaluated in double and rounded once, the
// angle of the CPU reference (src/qwen_ops.cpp:18-19; the tables of tests/rope_verify.cpp:73-81 are built the same
// way, on the host); pairs at or beyond rot_pairs get (1, 0). A forward pass fills them once and every layer's q/k
// call reads them, as the reference's rope_rotate_half takes host-built tables (src/rope_embedding.hip:18-37).
// PER (4 or 1) consecutive pairs per thread, half / PER threads per token, 256 / (half / PER) tokens per CTA pass.
template <bool FAST_TRIG, int PER>
__global__ void __launch_bounds__(256)
k_rope_table(const int* positions, int pos0, long long T, int half, int rot_pairs, const float* ff, float* cos_out,
             float* sin_out, const __grid_constant__ RopeFreq fr) {
    pdl_entry();
    __shared__ double invf[B200_MAX_ROT_PAIRS];
    stage_inv_freq(invf, fr, half);
    const int L = half / PER, tpp = 256 / L;
    const int l = threadIdx.x % L, slot = threadIdx.x / L;
    if (slot >= tpp) return;
    double f[PER];
    bool rot[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = l * PER + j;
        rot[j] = i < rot_pairs;
        f[j] = invf[i];
    }
    for (long long t = (long long)blockIdx.x * tpp + slot; t < T; t += (long long)gridDim.x * tpp) {
        const int pos = positions ? positions[t] : pos0 + (int)t;
        float c[PER], s[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            c[j] = 1.0f;
            s[j] = 0.0f;
            if (rot[j]) {
                double theta = (double)pos * f[j];
                if (ff) theta /= (double)ff[l * PER + j];
                double ds, dc;
                if (FAST_TRIG) sincos_cw(theta, &ds, &dc);   // (the launcher guarantees |theta| < 2^31 here)
                else sincos(theta, &ds, &dc);
                c[j] = (float)dc;
                s[j] = (float)ds;
            }
        }
        float* co = cos_out + (size_t)t * half + l * PER;
        float* so = sin_out + (size_t)t * half + l * PER;
        if constexpr (PER == 4) {
            *reinterpret_cast<float4*>(co) = make_float4(c[0], c[1], c[2], c[3]);
            *reinterpret_cast<float4*>(so) = make_float4(s[0], s[1], s[2], s[3]);
        } else {
            co[0] = c[0];
            so[0] = s[0];
        }
    }
}

}  // namespace b200

#endif  // B200_QK_NORM_ROPE_CUH
