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

}  // namespace b200

#endif  // B200_KV_STORE_CUH
