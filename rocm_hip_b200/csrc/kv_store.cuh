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

// Quantised cache rows (src/attention.hip:44-50, kvq_store :159-178): a row holds d_row values and then one fp16 scale
// per 32 values; d_row = kv_stride * 32 / 17 (Q8_0) or kv_stride * 32 / 9 (Q4_0), kv_stride still in fp16 units.
//   KQ 1, Q8_0: d = amax / 127; q = rint(x * (1 / d)) as int8 (0 when d == 0); scales start at byte d_row.
//   KQ 2, Q4_0: d = m / -8, m the value of largest magnitude (the positive one on a +- tie);
//               n = min(15, (int)(x * (1 / d) + 8.5)) (8 when d == 0); byte 4 j + k (k < 4) of the row holds value
//               8 j + k in its low and value 8 j + k + 4 in its high nibble; scales start at byte d_row / 2.
// The scale is stored rounded to fp16; the values are quantised with the unrounded d. Every operation rounds on its
// own. A warp owns a 32-value block, lane = value; a warp takes U blocks per step so U loads are in flight per lane.
template <typename IO, int KQ, int U>
__global__ void __launch_bounds__(256)
k_kv_store_q(const IO* src, __half* cache, int n_vals, const int* positions, int pos0, long long T, int kv_stride,
             int kv_shift, long long kv_bstride) {
    const int lane = threadIdx.x & 31;
    const int bpr = n_vals / 32;                      // blocks per row
    const long long nblk = T * bpr;
    const int d_row = kv_stride * 32 / (KQ == 2 ? 9 : 17);
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long b0 = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * U; b0 < nblk; b0 += warps * U) {
        float x[U];
#pragma unroll
        for (int j = 0; j < U; ++j) x[j] = b0 + j < nblk ? Io<IO>::load1(src + (b0 + j) * 32 + lane) : 0.0f;
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (b0 + j >= nblk) break;                // warp-uniform
            const long long t = (b0 + j) / bpr;
            const int blk = (int)(b0 + j - t * bpr);
            const int pos = positions ? positions[t] : pos0 + (int)t;
            uint8_t* row = reinterpret_cast<uint8_t*>(cache + kv_row(pos, kv_stride, kv_shift, kv_bstride));
            float amax = fabsf(x[j]);
            for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            if (KQ == 1) {
                const float d = __fdiv_rn(amax, 127.0f);
                const float q = d != 0.0f ? __fmul_rn(x[j], __fdiv_rn(1.0f, d)) : 0.0f;
                reinterpret_cast<int8_t*>(row)[blk * 32 + lane] = (int8_t)(int)rintf(q);
                if (lane == 0) reinterpret_cast<__half*>(row + d_row)[blk] = __float2half_rn(d);
            } else {
                float m = fabsf(x[j]) == amax ? x[j] : -INFINITY;
                for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
                const float d = __fdiv_rn(m, -8.0f);
                const int n = min(15, (int)(d != 0.0f ? __fadd_rn(__fmul_rn(x[j], __fdiv_rn(1.0f, d)), 8.5f) : 8.0f));
                const int hi = __shfl_down_sync(0xffffffffu, n, 4);
                if ((lane & 4) == 0) row[blk * 16 + (lane >> 3) * 4 + (lane & 3)] = (uint8_t)(n | (hi << 4));
                if (lane == 0) reinterpret_cast<__half*>(row + d_row / 2)[blk] = __float2half_rn(d);
            }
        }
    }
}

}  // namespace b200

#endif  // B200_KV_STORE_CUH
