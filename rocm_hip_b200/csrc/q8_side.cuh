// q8_side.cuh -- the producers' activation side outputs: the values of a finished output vector rounded to bf16 /
// fp16 and / or quantised to ggml's Q8_0 and Q8_K activation formats, as the reference's q8_block_value does inside
// its producer kernels (src/q8_device.h:54-104). Rules, bit for bit:
//   xh   : value rounded to bf16 (nearest even) or fp16
//   Q8_0 : per 32 values d = amax / 127 (stored fp16-rounded), q = rint(x * (127 / amax)), s0 = fp16(d * sum q) bits
//   Q8_K : per 256 values, max = the signed value of largest |x| (lowest index on ties), iscale = -127 / max,
//          q = min(127, rint(iscale * x)), d = 1 / iscale, plus the sum of every 16 q
// The int8 outputs are written only when qK is set (then q0, d0, s0, dK, bsK are all expected), xh only when set.
// A last partial 256-value block (n a multiple of 32 only) gets its Q8_0 part and an incomplete Q8_K part, as in the
// reference. Three forms: q8_block_value, one value per thread of a 256-thread group (the reference's shape, used by
// the by-name kernels); q8v_phase_a / q8v_phase_b, for a producer whose threads hold 16-byte vectors of the finished
// output (the norm and SwiGLU kernels write the side outputs themselves with it: one launch); and k_q8_side, a warp
// per block over a vector in memory (for the producers that cannot).

#ifndef B200_Q8_SIDE_CUH
#define B200_Q8_SIDE_CUH

#include "common.cuh"

namespace b200 {

// rint(t) (ties to even, as __float2int_rn) for |t| < 2^22: the sum t + 1.5 * 2^23 holds it in its low mantissa bits
// (two's complement), so the conversion is one add on the fp32 pipe instead of an instruction of the quarter-rate
// conversion unit, which these quantisers otherwise keep busiest. The quantisers' products are within +-127.5 for
// finite values; a vector with a non-finite value gets unspecified int8 values (the C conversion of an infinite
// product is undefined, so there is nothing to match there).
__device__ __forceinline__ int rint_small(float t) { return (int)__float_as_uint(__fadd_rn(t, 12582912.0f)) - 0x4B400000; }

// Four such values as the int8 quadruple a quantiser stores: the low byte of each sum is the value's two's-complement
// byte already (the constant's low byte is 0), so the four sums are packed without being turned into integers first;
// their integer sum is one dot product with four ones.
__device__ __forceinline__ uint32_t rint4_packed(float t0, float t1, float t2, float t3) {
    const uint32_t b0 = __float_as_uint(__fadd_rn(t0, 12582912.0f)), b1 = __float_as_uint(__fadd_rn(t1, 12582912.0f));
    const uint32_t b2 = __float_as_uint(__fadd_rn(t2, 12582912.0f)), b3 = __float_as_uint(__fadd_rn(t3, 12582912.0f));
    return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}
__device__ __forceinline__ int sum_int8x4(uint32_t packed) { return __dp4a((int)packed, 0x01010101, 0); }


struct Q8Side {
    int8_t* q0;
    float* d0;
    int8_t* qK;
    float* dK;
    int32_t* bsK;
    int32_t* s0;
    uint16_t* xh;
    int xh_bf16;
};

// Shared scratch of one 256-thread group
struct Q8Scratch {
    float a[8], v[8];
    int i[8];
};

// Side outputs of value v, element t (0..255) of 256-value block b of the flattened vector. Every thread of the
// 256-thread group calls it the same number of times (it synchronises the group twice); a thread past the end of the
// vector passes active = false.
__device__ __forceinline__ void q8_block_value(float v, bool active, long long b, int t, Q8Scratch& sh, const Q8Side& o) {
    const int lane = t & 31, w = t >> 5;
    const long long i = b * 256 + t;
    if (o.xh && active) o.xh[i] = o.xh_bf16 ? to_bf16_bits(v) : __half_as_ushort(__float2half_rn(v));
    if (!o.qK) return;  // uniform
    const float a = active ? fabsf(v) : 0.0f;

    float am = a;
    for (int off = 16; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
    const float id0 = am != 0.0f ? __fdiv_rn(127.0f, am) : 0.0f;
    const int q0 = active ? __float2int_rn(__fmul_rn(v, id0)) : 0;
    int sum0 = q0;
    for (int off = 16; off > 0; off >>= 1) sum0 += __shfl_xor_sync(0xffffffffu, sum0, off);
    if (active) {
        o.q0[i] = (int8_t)q0;
        if (lane == 0) {
            const float d = __fdiv_rn(am, 127.0f);
            o.d0[b * 8 + w] = __half2float(__float2half_rn(d));
            o.s0[b * 8 + w] = __float_as_int(__half2float(__float2half_rn(__fmul_rn(d, (float)sum0))));
        }
    }

    // largest |x| of the block, lowest index on ties
    float ba = a, bv = v;
    int bi = t;
    for (int off = 16; off > 0; off >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, ba, off), ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (oa > ba || (oa == ba && oi < bi)) { ba = oa; bi = oi; bv = ov; }
    }
    if (lane == 0) { sh.a[w] = ba; sh.i[w] = bi; sh.v[w] = bv; }
    __syncthreads();
    float fa = sh.a[0], fv = sh.v[0];
    int fi = sh.i[0];
#pragma unroll
    for (int k = 1; k < 8; ++k)
        if (sh.a[k] > fa || (sh.a[k] == fa && sh.i[k] < fi)) { fa = sh.a[k]; fi = sh.i[k]; fv = sh.v[k]; }
    __syncthreads();  // the scratch is reused by the next call
    int q = 0;
    float iscale = 0.0f;
    if (fa != 0.0f) {
        iscale = __fdiv_rn(-127.0f, fv);
        q = min(127, __float2int_rn(__fmul_rn(iscale, v)));
    }
    int s16 = q;
    for (int off = 8; off > 0; off >>= 1) s16 += __shfl_xor_sync(0xffffffffu, s16, off);
    if (active) {
        o.qK[i] = (int8_t)q;
        if (t == 0) o.dK[b] = fa != 0.0f ? __fdiv_rn(1.0f, iscale) : 0.0f;
        if ((lane & 15) == 0) o.bsK[b * 16 + w * 2 + (lane >> 4)] = s16;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same outputs written by a producer whose threads hold NV finished 16-byte vectors of 4 fp32 values each, the 32
// lanes of a warp holding 32 consecutive vectors per slot (the row kernels of rmsnorm.cuh, the tiles of swiglu.cuh): a
// Q8_0 block is 8 neighbouring lanes of a slot, a Q8_K block two neighbouring groups of 32 lanes. Built for the fewest
// instructions per value (the producers are bound by instruction issue once this is added):
//   * maxima are taken of the |x| bit patterns (they order like the values): one 32-bit shuffle and one integer
//     maximum per step, the Q8_0 block's maximum falling out after three steps, the warp's after five;
//   * which value holds a Q8_K block's maximum (lowest index on ties) and its sign is found without a second
//     reduction: the few lanes that hold the warp's maximum post index << 1 | sign with a shared-memory atomicMin;
//   * the IEEE divisions of the rules (127 / amax, amax / 127, -127 / max, 1 / iscale) are batched: a division costs
//     the warp its ~20 instructions whether one lane or all need it, so lane j (and NV + j) of a group divides for
//     slot j and the quotients travel by shuffle: 3 division sequences per thread instead of 4 per vector.
//     (Warp-reduce instructions, redux.sync, were measured 1.7x slower than the shuffle steps they replace.)
// q8v_phase_a writes the Q8_0 part and leaves, per slot, the maximum |x| bits of the warp's 128 values and the
// candidate code of the lowest index that has it in the slot's shared-memory cell; after a barrier the caller
// combines the cells of a block's two halves (q8v_combine) and q8v_phase_b writes the Q8_K part.
// Same rules and bits as q8_block_value and k_q8_side. NV <= 4.

struct Q8Half { unsigned am, cand; };

__device__ __forceinline__ Q8Half q8v_combine(Q8Half first, Q8Half second) {   // halves in index order
    Q8Half r;
    r.am = first.am > second.am ? first.am : second.am;
    r.cand = first.am > second.am ? first.cand : (second.am > first.am ? second.cand : min(first.cand, second.cand));
    return r;
}

// y[j]: slot j's 4 values, elements i[j] .. i[j] + 3 of the flattened vector (i[j] a multiple of 4; the warp's lanes
// hold i0 + 4 * lane; 32-bit: the reference's launchers bound the vector by an int, src/gpu_ops.cpp:70,82). live[j] false: the vector lies past the end (the 8 lanes of a Q8_0 block are live or dead
// together); its values count as zeros and nothing is stored for it. cell[j]: the warp's shared-memory cell of slot j.
template <int NV>
__device__ __forceinline__ void q8v_phase_a(const float (&y)[NV][4], const unsigned (&i)[NV], const bool (&live)[NV],
                                            const Q8Side& o, Q8Half* const (&cell)[NV]) {
    static_assert(NV <= 4, "lanes j and NV + j of an 8-lane group divide for slot j");
    const int lane = threadIdx.x & 31, r = lane & 7;
    unsigned am8[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        unsigned ab[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) ab[e] = live[j] ? (__float_as_uint(y[j][e]) & 0x7fffffffu) : 0u;
        unsigned t = max(max(ab[0], ab[1]), max(ab[2], ab[3]));
        t = max(t, __shfl_xor_sync(0xffffffffu, t, 1));
        t = max(t, __shfl_xor_sync(0xffffffffu, t, 2));
        t = max(t, __shfl_xor_sync(0xffffffffu, t, 4));
        am8[j] = t;
        t = max(t, __shfl_xor_sync(0xffffffffu, t, 8));
        t = max(t, __shfl_xor_sync(0xffffffffu, t, 16));
        if (lane == 0) { cell[j]->am = t; cell[j]->cand = 0xffffffffu; }
        __syncwarp();
        const unsigned in_blk = i[j] & 255u;
        unsigned c = 0xffffffffu;
#pragma unroll
        for (int e = 3; e >= 0; --e)
            if (ab[e] == t) c = ((in_blk + e) << 1) | (__float_as_uint(y[j][e]) >> 31);
        if (live[j] && c != 0xffffffffu) atomicMin(&cell[j]->cand, c);
    }
    // lane j of a group: 127 / amax of slot j; lane NV + j: amax / 127 (both 0 when amax is 0)
    float am = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (r == j || r == NV + j) am = __uint_as_float(am8[j]);
    const bool is_id = r < NV;
    const float quot = (r < 2 * NV && am != 0.0f) ? __fdiv_rn(is_id ? 127.0f : am, is_id ? am : 127.0f) : 0.0f;
    // lane NV + j of a group writes slot j's scale and scaled sum: its own slot-j values pick the block (same 32-value
    // block for all 8 lanes), and the writes are issued once, after the loop, instead of once per slot
    int my_sum = 0;
    unsigned my_i = 0u;
    bool my_live = false;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const float id0 = __shfl_sync(0xffffffffu, quot, (lane & 24) + j);
        const uint32_t q4 = live[j] ? rint4_packed(__fmul_rn(y[j][0], id0), __fmul_rn(y[j][1], id0), __fmul_rn(y[j][2], id0),
                                                   __fmul_rn(y[j][3], id0))
                                    : 0u;
        int sum0 = sum_int8x4(q4);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 4);
        if (live[j]) *reinterpret_cast<uint32_t*>(o.q0 + i[j]) = q4;
        if (r == NV + j) { my_sum = sum0; my_i = i[j]; my_live = live[j]; }
    }
    if (my_live) {   // (only lanes NV .. 2 NV - 1 of a group: this lane holds amax / 127 of its block in quot)
        o.d0[my_i >> 5] = __half2float(__float2half_rn(quot));
        o.s0[my_i >> 5] = __float_as_int(__half2float(__float2half_rn(__fmul_rn(quot, (float)my_sum))));
    }
}

// blk[j]: the combined halves of slot j's block. first_half[j]: this warp holds the block's first 128 values.
template <int NV>
__device__ __forceinline__ void q8v_phase_b(const float (&y)[NV][4], const unsigned (&i)[NV], const bool (&live)[NV],
                                            const Q8Side& o, const Q8Half (&blk)[NV], const bool (&first_half)[NV]) {
    const int lane = threadIdx.x & 31;
    // lane j: -127 / (the signed value of largest magnitude of slot j's block), then 1 / that
    unsigned ab = 0u, sg = 0u;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (lane == j) { ab = blk[j].am; sg = blk[j].cand & 1u; }
    const bool on = lane < NV && ab != 0u;
    const float isc = on ? __fdiv_rn(-127.0f, __uint_as_float(ab | (sg << 31))) : 0.0f;
    const float dk = on ? __fdiv_rn(1.0f, isc) : 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const float iscale = __shfl_sync(0xffffffffu, isc, j);
        // min(127, rint(t)) = rint(min(t, 127))
        const uint32_t q4 = (live[j] && blk[j].am != 0u)
                                ? rint4_packed(fminf(__fmul_rn(iscale, y[j][0]), 127.0f), fminf(__fmul_rn(iscale, y[j][1]), 127.0f),
                                               fminf(__fmul_rn(iscale, y[j][2]), 127.0f), fminf(__fmul_rn(iscale, y[j][3]), 127.0f))
                                : 0u;
        int s16 = sum_int8x4(q4);
        s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
        s16 += __shfl_xor_sync(0xffffffffu, s16, 2);
        if (live[j]) {
            *reinterpret_cast<uint32_t*>(o.qK + i[j]) = q4;
            if ((lane & 3) == 0) o.bsK[i[j] >> 4] = s16;
            if (lane == j && first_half[j]) o.dK[i[j] >> 8] = dk;
        }
    }
}

// The same outputs for a finished vector in memory, at memory speed: one warp per 256-value block, a lane owns 8
// consecutive values (two 16-byte loads; its int8 results are one 8-byte store per format, its 16-bit copy one 16-byte
// store), a Q8_0 block is four neighbouring lanes, a Q8_K block the warp, so every reduction is a shuffle. Same rules
// and the same bits as q8_block_value (which keeps the reference's one-value-per-thread shape for kernels that call
// it on a value in flight). With qK set K is a multiple of 32, so a lane's 8 values are all inside or all outside.
// VEC: x, q0, qK 16- / 8-byte aligned and xh 16-byte aligned.
template <bool VEC>
__global__ void __launch_bounds__(256)
k_q8_side(const float* x, long long K, Q8Side o) {
    const int lane = threadIdx.x & 31;
    const long long nblk = (K + 255) / 256;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblk; b += warps) {
        const long long i = b * 256 + lane * 8;
        const int act = (int)(K - i >= 8 ? 8 : (K - i > 0 ? K - i : 0));      // live values of this lane
        float v[8];
        if (VEC && act == 8) {
            Io<float>::unpack(ld_stream(x + i), v);
            Io<float>::unpack(ld_stream(x + i + 4), v + 4);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = e < act ? x[i + e] : 0.0f;
        }
        if (o.xh) {
            if (VEC && act == 8) {
                const uint4 r = o.xh_bf16 ? Io<__nv_bfloat16>::pack(v) : Io<__half>::pack(v);
                st_stream(o.xh + i, r);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (e < act) o.xh[i + e] = o.xh_bf16 ? to_bf16_bits(v[e]) : __half_as_ushort(__float2half_rn(v[e]));
            }
        }
        if (!o.qK) continue;  // uniform
        const bool active = act == 8;

        // Q8_0: 32 values = lanes 4 g .. 4 g + 3
        float am = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) am = fmaxf(am, fabsf(v[e]));
        float ba = 0.0f, bv = 0.0f;      // this lane's largest |x| and its signed value, lowest index on ties
        int bi = lane * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (fabsf(v[e]) > ba || e == 0) { ba = fabsf(v[e]); bv = v[e]; bi = lane * 8 + e; }
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        const float id0 = am != 0.0f ? __fdiv_rn(127.0f, am) : 0.0f;
        int q[8], sum0 = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) { q[e] = rint_small(__fmul_rn(v[e], id0)); sum0 += q[e]; }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        if (active) {
            uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
            for (int e = 0; e < 4; ++e) { w0 |= (uint32_t)(q[e] & 0xff) << (8 * e); w1 |= (uint32_t)(q[e + 4] & 0xff) << (8 * e); }
            if (VEC) *reinterpret_cast<uint2*>(o.q0 + i) = make_uint2(w0, w1);
            else {
#pragma unroll
                for (int e = 0; e < 8; ++e) o.q0[i + e] = (int8_t)q[e];
            }
            if ((lane & 3) == 0) {
                const float d = __fdiv_rn(am, 127.0f);
                o.d0[b * 8 + (lane >> 2)] = __half2float(__float2half_rn(d));
                o.s0[b * 8 + (lane >> 2)] = __float_as_int(__half2float(__float2half_rn(__fmul_rn(d, (float)sum0))));
            }
        }

        // Q8_K: the warp's 256 values
        for (int off = 16; off > 0; off >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, ba, off), ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (oa > ba || (oa == ba && oi < bi)) { ba = oa; bi = oi; bv = ov; }
        }
        float iscale = 0.0f;
        int s8 = 0;
        if (ba != 0.0f) {
            iscale = __fdiv_rn(-127.0f, bv);
#pragma unroll
            for (int e = 0; e < 8; ++e) { q[e] = rint_small(fminf(__fmul_rn(iscale, v[e]), 127.0f)); s8 += q[e]; }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) q[e] = 0;
        }
        const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
        if (active) {
            uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
            for (int e = 0; e < 4; ++e) { w0 |= (uint32_t)(q[e] & 0xff) << (8 * e); w1 |= (uint32_t)(q[e + 4] & 0xff) << (8 * e); }
            if (VEC) *reinterpret_cast<uint2*>(o.qK + i) = make_uint2(w0, w1);
            else {
#pragma unroll
                for (int e = 0; e < 8; ++e) o.qK[i + e] = (int8_t)q[e];
            }
            if (lane == 0) o.dK[b] = ba != 0.0f ? __fdiv_rn(1.0f, iscale) : 0.0f;
            if ((lane & 1) == 0) o.bsK[b * 16 + (lane >> 1)] = s16;
        }
    }
}

}  // namespace b200

#endif  // B200_Q8_SIDE_CUH
