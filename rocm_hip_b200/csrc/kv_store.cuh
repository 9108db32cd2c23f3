// kv_store.cuh -- writes K / V rows into the block-major FP16 KV cache, the epilogue of the reference's attn_prep
// kernels for an unquantised cache (src/attention.hip:279-300, F16 branch :296-299). Row of position p, in __half
// units from the layer's row 0 (src/attention.hip:38-42, layout src/kv_cache.h:7-14):
//   (p >> kv_shift) * kv_bstride + (p & ((1 << kv_shift) - 1)) * kv_stride      (a contiguous cache: kv_shift = 30)
// Token t of the batch sits at positions[t], or pos0 + t. Values are rounded to fp16 once (round to nearest even, as
// __float2half). Per token: n_vals * s bytes read, n_vals * 2 written.

#ifndef B200_KV_STORE_CUH
#define B200_KV_STORE_CUH

#include "common.cuh"

namespace b200 {

__device__ __forceinline__ size_t kv_row(int p, int kv_stride, int kv_shift, long long kv_bstride) {
    return (size_t)(p >> kv_shift) * (size_t)kv_bstride + (size_t)(p & ((1 << kv_shift) - 1)) * (size_t)kv_stride;
}

// VEC: n_vals a multiple of 8, src rows and cache rows 16-byte aligned: a thread converts 8 values per step
template <typename IO, bool VEC>
__global__ void __launch_bounds__(256)
k_kv_store_f16(const IO* src, __half* cache, int n_vals, const int* positions, int pos0, long long T, int kv_stride,
               int kv_shift, long long kv_bstride) {
    const int per_row = VEC ? n_vals / 8 : n_vals;
    const long long total = T * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per_row;
        const int c = (int)(i - t * per_row);
        const int pos = positions ? positions[t] : pos0 + (int)t;
        __half* row = cache + kv_row(pos, kv_stride, kv_shift, kv_bstride);
        const IO* s = src + (size_t)t * n_vals;
        if (VEC) {
            float v[8];
            if (sizeof(IO) == 4) {
                Io<float>::unpack(ld_stream(reinterpret_cast<const float*>(s) + c * 8), v);
                Io<float>::unpack(ld_stream(reinterpret_cast<const float*>(s) + c * 8 + 4), v + 4);
            } else {
                Io<__nv_bfloat16>::unpack(ld_stream(reinterpret_cast<const __nv_bfloat16*>(s) + c * 8), v);
            }
            st_stream(row + c * 8, Io<__half>::pack(v));
        } else {
            row[c] = __float2half_rn(Io<IO>::load1(s + c));
        }
    }
}

// Orthonormal Walsh-Hadamard transform of blocks of N values (N = 64, 128, 256 or 512), as the reference rotates q, K
// and V for a quantised cache (hadamard_rot, src/attention.hip:238-263): stages s = 1, 2, ..., N / 2 in that order,
// value d becoming (d & s) ? v[d ^ s] - v[d] : v[d] + v[d ^ s], then one multiply by 1 / sqrt(N). A lane holds values
// 8 lane .. 8 lane + 7 of its warp's 256: stages below 8 stay inside the lane, stages up to 128 are one shuffle per
// value, and the last stage of a 512-block pairs two neighbouring warps of the CTA through shared memory (xchg:
// 8 * blockDim.x floats; the pair meets at its own named barrier, so other warps may have left the kernel). Same
// operations in the same order as the reference's shared-memory butterflies, so the same bits.
// Callers keep 256-value chunks on consecutive warps: thread t of the CTA holds octet (CTA base + t).
__device__ __forceinline__ void wht8(float (&x)[8], int N, float* xchg) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = (e & s) ? __fsub_rn(x[e ^ s], x[e]) : __fadd_rn(x[e], x[e ^ s]);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = y[e];
    }
    const int in_warp = N < 256 ? N / 8 : 32;
    for (int s = 1; s < in_warp; s <<= 1) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float y = __shfl_xor_sync(0xffffffffu, x[e], s);
            x[e] = (lane & s) ? __fsub_rn(y, x[e]) : __fadd_rn(x[e], y);
        }
    }
    if (N == 512) {   // uniform
        const int warp = threadIdx.x >> 5, bar = 1 + (warp >> 1);
#pragma unroll
        for (int e = 0; e < 8; ++e) xchg[e * blockDim.x + threadIdx.x] = x[e];
        asm volatile("bar.sync %0, 64;" ::"r"(bar) : "memory");
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float y = xchg[e * blockDim.x + (threadIdx.x ^ 32)];
            x[e] = (warp & 1) ? __fsub_rn(y, x[e]) : __fadd_rn(x[e], y);
        }
        asm volatile("bar.sync %0, 64;" ::"r"(bar) : "memory");   // the buffer is written again on the next step
    }
    const float r = __fdiv_rn(1.0f, __fsqrt_rn((float)N));
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = __fmul_rn(x[e], r);
}

// The quantisers' float -> int conversions without the conversion unit (a quarter-rate pipe that these kernels keep
// busiest): for |t| < 2^22 the sum t + 1.5 * 2^23, rounded to nearest even, holds rint(t) in its low mantissa bits
// (two's complement), exactly what __float2int_rn gives; for 0 <= u < 2^23 the sum u + 2^23 rounded DOWN holds
// floor(u) = (int)u. The products of a block of finite values lie within [-127.001, 127.001] and [0.49, 16.51]. A
// block with a non-finite value, or with a scale too small to invert in fp32, stores unspecified (in-range) bytes: the
// C conversion of an infinite product is undefined, so there is nothing to match there.
__device__ __forceinline__ uint32_t rint_low_bits(float t) { return __float_as_uint(__fadd_rn(t, 12582912.0f)); }
__device__ __forceinline__ uint32_t floor_low_bits(float u) { return __float_as_uint(__fadd_rd(u, 8388608.0f)); }

// Q4_0's scale source: the value of largest magnitude, the positive one on a +- tie (src/attention.hip:169-171), from
// the block's largest and smallest value: the largest if it is at least as far from zero as the smallest, else the
// smallest. (A block of zeros: max(+0, -0) is +0 whatever the order, as in the reference's max over the candidates.)
__device__ __forceinline__ float q4_0_extreme(float vmax, float vmin) { return vmax >= -vmin ? vmax : vmin; }

// Quantised cache rows (src/attention.hip:44-50, kvq_store :159-178): a row holds d_row values and then one fp16 scale
// per 32 values; d_row = kv_stride * 32 / 17 (Q8_0) or kv_stride * 32 / 9 (Q4_0), kv_stride still in fp16 units.
//   KQ 1, Q8_0: d = amax / 127; q = rint(x * (1 / d)) as int8 (0 when d == 0); scales start at byte d_row.
//   KQ 2, Q4_0: d = m / -8, m the value of largest magnitude (the positive one on a +- tie);
//               n = min(15, (int)(x * (1 / d) + 8.5)) (8 when d == 0); byte 4 j + k (k < 4) of the row holds value
//               8 j + k in its low and value 8 j + k + 4 in its high nibble; scales start at byte d_row / 2.
// The scale is stored rounded to fp16; the values are quantised with the unrounded d. Every operation rounds on its
// own. A thread owns 8 consecutive values (32 or 16 bytes read, 8 or 4 bytes written: for Q4_0 its eight values are
// exactly one 32-bit word of the row), four neighbouring lanes own a block and share its maximum with two shuffles.
// U octets per thread and step are loaded before the first is used. rot = 64, 128, 256 or 512: the values are rotated in
// blocks of rot (wht8) before they are quantised, attn_prep's ATTN_KV_ROT (src/attention.hip:290-293).
template <typename IO, int KQ, int U, bool ROT>
__global__ void __launch_bounds__(256)
k_kv_store_q(const IO* src, __half* cache, int n_vals, const int* positions, int pos0, long long T, int kv_stride,
             int kv_shift, long long kv_bstride, int rot) {
    __shared__ float xchg[ROT ? 8 * 256 : 1];
    const int opr = n_vals / 8;                       // octets per row
    const long long total = T * opr;
    const int d_row = kv_stride * 32 / (KQ == 2 ? 9 : 17);
    const long long stride = (long long)gridDim.x * blockDim.x;
    // every lane of a warp runs the same number of steps (the shuffles need all four lanes of a block; a block
    // never straddles the end because n_vals is a multiple of 32)
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 - threadIdx.x % 32 < total; i0 += stride * U) {
        float x[U][8];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const long long i = i0 + j * stride;
            if (i < total) {
                if (sizeof(IO) == 4) {
                    Io<float>::unpack(ld_stream(reinterpret_cast<const float*>(src) + i * 8), x[j]);
                    Io<float>::unpack(ld_stream(reinterpret_cast<const float*>(src) + i * 8 + 4), x[j] + 4);
                } else {
                    Io<__nv_bfloat16>::unpack(ld_stream(reinterpret_cast<const __nv_bfloat16*>(src) + i * 8), x[j]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[j][e] = 0.0f;
            }
        }
        if (ROT) {   // rotate in blocks of rot values first (n_vals % rot == 0, so a block is whole)
#pragma unroll
            for (int j = 0; j < U; ++j) wht8(x[j], rot, xchg);
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const long long i = i0 + j * stride;
            const bool live = i < total;
            // the block's extremes over its four lanes: Q8_0 needs the largest magnitude, Q4_0 the largest and the
            // smallest value (q4_0_extreme)
            float amax = 0.0f, vmax = x[j][0], vmin = x[j][0];
            if (KQ == 1) {
#pragma unroll
                for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(x[j][e]));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            } else {
#pragma unroll
                for (int e = 1; e < 8; ++e) { vmax = fmaxf(vmax, x[j][e]); vmin = fminf(vmin, x[j][e]); }
                vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 1));
                vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, 1));
                vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 2));
                vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, 2));
            }
            if (!live) continue;
            const long long t = i / opr;
            const int o = (int)(i - t * opr);            // octet of the row; block o / 4
            const int pos = positions ? positions[t] : pos0 + (int)t;
            uint8_t* row = reinterpret_cast<uint8_t*>(cache + kv_row(pos, kv_stride, kv_shift, kv_bstride));
            if (KQ == 1) {
                const float d = __fdiv_rn(amax, 127.0f);
                const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                uint32_t w[2] = {0u, 0u};
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    w[e >> 2] |= (rint_low_bits(__fmul_rn(x[j][e], id)) & 0xffu) << (8 * (e & 3));
                *reinterpret_cast<uint2*>(row + o * 8) = make_uint2(w[0], w[1]);
                if ((o & 3) == 0) reinterpret_cast<__half*>(row + d_row)[o >> 2] = __float2half_rn(d);
            } else {
                const float d = __fdiv_rn(q4_0_extreme(vmax, vmin), -8.0f);
                const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                uint32_t w = 0u;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t n = floor_low_bits(fminf(__fadd_rn(__fmul_rn(x[j][e], id), 8.5f), 15.5f)) & 0xfu;
                    w |= n << (8 * (e & 3) + 4 * (e >> 2));     // value e: byte e % 4, high nibble for e >= 4
                }
                *reinterpret_cast<uint32_t*>(row + o * 4) = w;
                if ((o & 3) == 0) reinterpret_cast<__half*>(row + d_row / 2)[o >> 2] = __float2half_rn(d);
            }
        }
    }
}

// One Q8_0 block (values, scale) from 32 finished values of a lane. Returns d.
__device__ __forceinline__ float q8_0_block_words(const float (&x)[32], uint32_t (&w)[8]) {
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(x[e]));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        w[j] = 0u;
#pragma unroll
        for (int e = 0; e < 4; ++e) w[j] |= (rint_low_bits(__fmul_rn(x[4 * j + e], id)) & 0xffu) << (8 * e);
    }
    return d;
}

// One Q4_0 block from 32 finished values of a lane: word j holds values 8 j .. 8 j + 7, byte k = value k (low nibble)
// and k + 4 (high). Returns d. (d == 0: id = 0, every value stores floor(8.5) = 8, as the reference's 8.0f.)
__device__ __forceinline__ float q4_0_block_words(const float (&x)[32], uint32_t (&w)[4]) {
    float vmax = x[0], vmin = x[0];
#pragma unroll
    for (int e = 1; e < 32; ++e) { vmax = fmaxf(vmax, x[e]); vmin = fminf(vmin, x[e]); }
    const float d = __fdiv_rn(q4_0_extreme(vmax, vmin), -8.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        w[j] = 0u;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t n = floor_low_bits(fminf(__fadd_rn(__fmul_rn(x[8 * j + e], id), 8.5f), 15.5f)) & 0xfu;
            w[j] |= n << (8 * (e & 3) + 4 * (e >> 2));
        }
    }
    return d;
}

// The 32 blocks (of 32 values) a warp owns in one step, from global memory into the lanes: lane l gets block l in
// x[0..31]. The warp reads its 4 KB (fp32) or 2 KB (16-bit) as consecutive 16-byte chunks, lane after lane, parks
// them in its 4 KB of shared memory and each lane picks its block's chunks up from there. Chunk c of the span belongs
// to lane c / CB (CB chunks per block) and is stored at chunk index c ^ s(owner), s chosen so that both the 8 lanes of
// a store phase and the 8 lanes of a load phase hit 8 different 16-byte bank groups. Blocks at or beyond n_live
// (counted from the warp's first block) read as zeros.
template <typename IO>
__device__ __forceinline__ void warp_blocks_load(const IO* src, long long first_block, long long n_live, float (&x)[32],
                                                 uint4* tile) {
    constexpr int CB = sizeof(IO) == 4 ? 8 : 4;   // 16-byte chunks per block
    const int lane = threadIdx.x & 31;
    const uint4* g = reinterpret_cast<const uint4*>(src) + first_block * CB;
    uint4 v[CB];
#pragma unroll
    for (int j = 0; j < CB; ++j) {
        const int c = lane + 32 * j;
        v[j] = (c / CB) < n_live ? ld_stream(g + c) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < CB; ++j) {
        const int c = lane + 32 * j, owner = c / CB;
        tile[c ^ (CB == 8 ? (owner & 7) : ((owner >> 1) & 3))] = v[j];
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < CB; ++k) {
        const uint4 r = tile[(CB * lane + k) ^ (CB == 8 ? (lane & 7) : ((lane >> 1) & 3))];
        if (sizeof(IO) == 4) Io<float>::unpack(r, x + 4 * k);
        else Io<__nv_bfloat16>::unpack(r, x + 8 * k);
    }
    __syncwarp();   // the tile is written again on the next step
}

// The way back: lane l's finished block, packed as CB chunks, through the same swizzled tile into consecutive chunks
// of global memory.
template <typename IO>
__device__ __forceinline__ void warp_blocks_store(IO* dst, long long first_block, long long n_live, const float (&x)[32],
                                                  uint4* tile) {
    constexpr int CB = sizeof(IO) == 4 ? 8 : 4;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 0; k < CB; ++k) {
        uint4 r;
        if (sizeof(IO) == 4) r = Io<float>::pack(x + 4 * k);
        else r = Io<__nv_bfloat16>::pack(x + 8 * k);
        tile[(CB * lane + k) ^ (CB == 8 ? (lane & 7) : ((lane >> 1) & 3))] = r;
    }
    __syncwarp();
    uint4* g = reinterpret_cast<uint4*>(dst) + first_block * CB;
#pragma unroll
    for (int j = 0; j < CB; ++j) {
        const int c = lane + 32 * j, owner = c / CB;
        const uint4 v = tile[c ^ (CB == 8 ? (owner & 7) : ((owner >> 1) & 3))];
        if (owner < n_live) st_stream(g + c, v);
    }
    __syncwarp();
}

// The transform of wht8 on a lane's whole block of 32 values: stages 1 .. 16 inside the lane, stages 32 .. N / 2 one
// shuffle per value between the N / 32 neighbouring lanes of a rotation block. Same operations in the same order per
// value as the reference's butterflies (src/attention.hip:251-263), so the same bits.
__device__ __forceinline__ void wht32(float (&x)[32], int N) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        float y[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) y[e] = (e & s) ? __fsub_rn(x[e ^ s], x[e]) : __fadd_rn(x[e], x[e ^ s]);
#pragma unroll
        for (int e = 0; e < 32; ++e) x[e] = y[e];
    }
    for (int s = 1; s < N / 32; s <<= 1) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
            const float y = __shfl_xor_sync(0xffffffffu, x[e], s);
            x[e] = (lane & s) ? __fsub_rn(y, x[e]) : __fadd_rn(x[e], y);
        }
    }
    const float r = __fdiv_rn(1.0f, __fsqrt_rn((float)N));
#pragma unroll
    for (int e = 0; e < 32; ++e) x[e] = __fmul_rn(x[e], r);
}

// out = the transform of x in blocks of N (64 .. 512): a lane per 32 values, global memory read and written as the
// warp's consecutive chunks (warp_blocks_load / _store). n_total a multiple of N.
template <typename IO>
__global__ void __launch_bounds__(128)
k_hadamard_rot32(const IO* x, IO* out, long long n_total, int N) {
    __shared__ uint4 tiles[4][256];
    const int lane = threadIdx.x & 31;
    const long long nblk = n_total / 32, stride = (long long)gridDim.x * blockDim.x;
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b - lane < nblk; b += stride) {
        float v[32];
        warp_blocks_load<IO>(x, b - lane, nblk - (b - lane), v, tiles[threadIdx.x >> 5]);
        wht32(v, N);
        warp_blocks_store<IO>(out, b - lane, nblk - (b - lane), v, tiles[threadIdx.x >> 5]);
    }
}

// The same rows with a lane owning a whole 32-value block (128 or 64 bytes read through L1, 32 or 16 bytes written as
// 16-byte vectors; fetching the warp's span as consecutive chunks and handing the blocks out through shared memory
// measured 0.41 against 0.57 rotated and 0.53 against 0.98 for 16-bit Q8_0 rows: L1 serves a lane's run well): the block maximum needs no shuffle, and a rotation block of rot values is rot / 32 neighbouring
// lanes, so only the stages from 32 up cross lanes (two shuffles per value at rot = 128 where the 8-per-lane form
// needs four). Same operations in the same order per value, so the same bits. Needs rows that start on 16 bytes. The
// launcher uses it for rotated rows and for 16-bit sources, where it is the faster of the two.
template <typename IO, int KQ, bool ROT, bool COAL = false>
__global__ void __launch_bounds__(128)
k_kv_store_q32(const IO* src, __half* cache, int n_vals, const int* positions, int pos0, long long T, int kv_stride,
               int kv_shift, long long kv_bstride, int rot) {
    const int lane = threadIdx.x & 31, bpr = n_vals / 32;
    const long long nblk = T * bpr, stride = (long long)gridDim.x * blockDim.x;
    const int d_row = kv_stride * 32 / (KQ == 2 ? 9 : 17);
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b - lane < nblk; b += stride) {
        const bool live = b < nblk;
        float x[32];
        if (COAL) {
            __shared__ uint4 tiles[COAL ? 4 : 1][COAL ? 256 : 1];
            warp_blocks_load<IO>(src, b - lane, nblk - (b - lane), x, tiles[threadIdx.x >> 5]);
        } else if (live) {
            if (sizeof(IO) == 4) {
#pragma unroll
                for (int j = 0; j < 8; ++j) Io<float>::unpack(__ldg(reinterpret_cast<const uint4*>(src) + b * 8 + j), x + 4 * j);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    Io<__nv_bfloat16>::unpack(__ldg(reinterpret_cast<const uint4*>(src) + b * 4 + j), x + 8 * j);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = 0.0f;
        }
        if (ROT) wht32(x, rot);
        if (!live) continue;
        const long long t = b / bpr;
        const int blk = (int)(b - t * bpr);
        const int pos = positions ? positions[t] : pos0 + (int)t;
        uint8_t* row = reinterpret_cast<uint8_t*>(cache + kv_row(pos, kv_stride, kv_shift, kv_bstride));
        if (KQ == 1) {
            uint32_t w[8];
            const float d = q8_0_block_words(x, w);
            uint4* o = reinterpret_cast<uint4*>(row + blk * 32);
            o[0] = make_uint4(w[0], w[1], w[2], w[3]);
            o[1] = make_uint4(w[4], w[5], w[6], w[7]);
            reinterpret_cast<__half*>(row + d_row)[blk] = __float2half_rn(d);
        } else {
            uint32_t w[4];
            const float d = q4_0_block_words(x, w);
            *reinterpret_cast<uint4*>(row + blk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<__half*>(row + d_row / 2)[blk] = __float2half_rn(d);
        }
    }
}

}  // namespace b200

#endif  // B200_KV_STORE_CUH
