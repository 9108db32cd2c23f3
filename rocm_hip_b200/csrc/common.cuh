// common.cuh -- shared device helpers for the sm_100a layer-op kernels: 16-byte streaming loads / stores, storage
// type traits (fp32, bf16, fp16 rows computed in fp32), and the fixed-order reductions.
//
// Rows are streamed once, so activation loads and stores bypass L1 allocation (the gammas, which every row
// re-reads, go through the read-only path and stay cached). Reductions always run in the same order for a given
// row width and storage type, independent of how many rows a launch holds or how the grid is shaped, so a row
// gives the same bits whether it is processed alone, in a batch, or on another GPU of a row-sharded run.

#ifndef B200_COMMON_CUH
#define B200_COMMON_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------- 16-byte global access

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// ---------------------------------------------------------------- asynchronous copies into shared memory
//
// Two forms. cp_async16: one 16-byte copy per thread and instruction, completion by cp.async.wait_group in the issuing
// thread. bulk_g2s: ONE instruction copies a whole contiguous run (a 16-byte aligned source and destination, a
// multiple of 16 bytes) through the copy engine and signals an mbarrier with the bytes written; no registers, no
// per-thread address arithmetic. Sources are always this GPU's own memory and no copy is multicast.
// Every wait on an mbarrier is bounded: mbar_wait gives up after a fixed number of polls and reports it, so a copy
// that never lands cannot hang the device.

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void cp_async_wait_all() {
    cp_async_commit();
    cp_async_wait<0>();
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// makes the initialised barriers visible to the copy engine
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// orders this thread's earlier shared-memory accesses before copy-engine writes it starts afterwards
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One thread: arms the barrier for `bytes` and starts the copy of `bytes` from global src to shared dst
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    const unsigned b = smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(b)
                 : "memory");
}

// Waits until the barrier's phase of the given parity has completed; false after MBAR_POLLS unsuccessful polls
#define MBAR_POLLS (1 << 18)
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned b = smem_u32(bar);
    for (int i = 0; i < MBAR_POLLS; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(b), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}

// ---------------------------------------------------------------- storage types

// bf16 <-> fp32. Widening is exact; narrowing is round-to-nearest-even, the same rule as the integer formula
// (u + 0x7fff + ((u >> 16) & 1)) >> 16 of the reference's half_bits (src/q8_device.h:39-40) for every finite value.
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint16_t to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <typename T>
struct Io;

template <>
struct Io<float> {
    static constexpr int VE = 4;  // values per 16-byte vector
    __device__ static __forceinline__ void unpack(const uint4& r, float* v) {
        v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y);
        v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
    }
    __device__ static __forceinline__ uint4 pack(const float* v) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
    __device__ static __forceinline__ float load1(const float* p) { return *p; }
    __device__ static __forceinline__ void store1(float* p, float v) { *p = v; }
    // value as it reads back after being stored
    __device__ static __forceinline__ float round_trip(float v) { return v; }
};

template <>
struct Io<__nv_bfloat16> {
    static constexpr int VE = 8;
    __device__ static __forceinline__ void unpack(const uint4& r, float* v) {
        v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x); v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
        v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z); v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
    }
    __device__ static __forceinline__ uint4 pack(const float* v) {
        return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    }
    __device__ static __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ static __forceinline__ void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
    __device__ static __forceinline__ float round_trip(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

template <>
struct Io<__half> {
    static constexpr int VE = 8;
    __device__ static __forceinline__ void unpack(const uint4& r, float* v) {
        const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ static __forceinline__ uint4 pack(const float* v) {
        return make_uint4(pack_f16(v[0], v[1]), pack_f16(v[2], v[3]), pack_f16(v[4], v[5]), pack_f16(v[6], v[7]));
    }
    __device__ static __forceinline__ float load1(const __half* p) { return __half2float(*p); }
    __device__ static __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
    __device__ static __forceinline__ float round_trip(float v) { return __half2float(__float2half_rn(v)); }
};

// ---------------------------------------------------------------- packed fp32 pairs
//
// sm_100 has two-wide fp32 instructions (add / sub / mul / fma .f32x2 on a 64-bit register holding two floats). Each
// lane rounds to nearest exactly like the scalar instruction, so results are bit-identical, at half the instruction
// count: these kernels are bound by instruction issue long before arithmetic throughput.
typedef unsigned long long f2;

__device__ __forceinline__ f2 pk2(float a, float b) { f2 r; asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void upk2(f2 v, float& a, float& b) { asm("mov.b64 {%0,%1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f2 mul2(f2 a, f2 b) { f2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) { f2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
__device__ __forceinline__ f2 add2(f2 a, f2 b) { f2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f2 sub2(f2 a, f2 b) { f2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }

// A 16-byte vector of stored values as VE / 2 packed pairs, and back (one rounding to the storage type)
template <typename T>
struct Io2;

template <>
struct Io2<float> {
    static constexpr int NP = 2;
    __device__ static __forceinline__ void unpack(const uint4& r, f2* v) {
        v[0] = ((f2)r.y << 32) | r.x;
        v[1] = ((f2)r.w << 32) | r.z;
    }
    __device__ static __forceinline__ uint4 pack(const f2* v) {
        return make_uint4((uint32_t)v[0], (uint32_t)(v[0] >> 32), (uint32_t)v[1], (uint32_t)(v[1] >> 32));
    }
};

template <>
struct Io2<__nv_bfloat16> {
    static constexpr int NP = 4;
    __device__ static __forceinline__ void unpack(const uint4& r, f2* v) {
        v[0] = pk2(bf16_lo(r.x), bf16_hi(r.x));
        v[1] = pk2(bf16_lo(r.y), bf16_hi(r.y));
        v[2] = pk2(bf16_lo(r.z), bf16_hi(r.z));
        v[3] = pk2(bf16_lo(r.w), bf16_hi(r.w));
    }
    __device__ static __forceinline__ uint32_t pack1(f2 v) {
        float a, b;
        upk2(v, a, b);
        return pack_bf16(a, b);
    }
    __device__ static __forceinline__ uint4 pack(const f2* v) {
        return make_uint4(pack1(v[0]), pack1(v[1]), pack1(v[2]), pack1(v[3]));
    }
};

// Four fp32 values (two packed pairs) rounded to bf16 or fp16 and stored as one 8-byte vector
__device__ __forceinline__ void st_half4(uint16_t* p, f2 v01, f2 v23, int bf16) {
    float a, b, c, d;
    upk2(v01, a, b);
    upk2(v23, c, d);
    const uint2 r = bf16 ? make_uint2(pack_bf16(a, b), pack_bf16(c, d)) : make_uint2(pack_f16(a, b), pack_f16(c, d));
    asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(r.x), "r"(r.y) : "memory");
}

// sum += a^2 + b^2 of a packed pair, in double
__device__ __forceinline__ void sumsq2(f2 v, double& s0, double& s1) {
    float a, b;
    upk2(v, a, b);
    s0 = fma((double)a, (double)a, s0);
    s1 = fma((double)b, (double)b, s1);
}

// gamma values for one vector of VE consecutive columns starting at column c (fp32 or fp16 gammas; NULL: all 1)
template <int VE, typename WT>
__device__ __forceinline__ void load_gamma(const WT* w, int c, float* g) {
    if (!w) {
#pragma unroll
        for (int i = 0; i < VE; ++i) g[i] = 1.0f;
        return;
    }
    if constexpr (sizeof(WT) == 4) {
#pragma unroll
        for (int i = 0; i < VE; i += 4) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(w + c + i));
            g[i] = f.x; g[i + 1] = f.y; g[i + 2] = f.z; g[i + 3] = f.w;
        }
    } else {
        static_assert(VE == 8, "16-bit gammas come with 16-bit rows");
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(w + c));
        Io<WT>::unpack(r, g);
    }
}

template <typename WT>
__device__ __forceinline__ float gamma1(const WT* w, int c) {
    if (!w) return 1.0f;
    if constexpr (sizeof(WT) == 4) return __ldg(w + c);
    else return Io<WT>::load1(w + c);
}

// ---------------------------------------------------------------- programmatic dependent launch
// First statement of the kernels a layer runs back to back. griddepcontrol.wait returns once the kernel before this
// one in the stream has completed and its writes are visible (at once if this kernel was launched the plain way);
// launch_dependents then lets the kernel after this one begin its own launch while this one runs, so that its CTAs
// are resident and waiting when this one's last CTAs retire: the launch latency between two short kernels (a decode
// step's are a few microseconds each) is hidden. Nothing is read or written before the wait, so no ordering changes.
__device__ __forceinline__ void pdl_entry() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- reductions

// Sum over the `width` lanes (a power of two <= 32) of an aligned lane group; every lane of the group gets the total.
// All 32 lanes of the warp must call it. Sums of squares are carried in double, as the CPU reference does
// (src/qwen_ops.cpp:9-10): on a bandwidth-bound kernel it is free, and it makes 1/rms the reference's to the bit.
__device__ __forceinline__ double group_sum(double v, int width) {
    for (int off = width >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Sum over all threads of the CTA (blockDim.x a multiple of 32, at most 1024). part: 32 doubles of shared memory
// that no other use touches between two calls with the same buffer.
__device__ __forceinline__ double cta_sum(double v, double* part) {
    v = group_sum(v, 32);
    const int nw = blockDim.x >> 5;
    if (nw == 1) return v;
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    double tot = 0.0;
    for (int k = 0; k < nw; ++k) tot += part[k];
    return tot;
}

// (float)(1 / sqrt(sum_sq / n + eps)), the CPU reference's double-precision expression (src/qwen_ops.cpp:11), without
// its ~70-instruction double division and square root: the hardware's single-precision rsqrt seeds two Newton steps in
// double (relative error 2^-22 -> 2^-44 -> below 2^-52), so the float it rounds to is the reference's unless the exact
// value lies within a few double ulps of a float rounding boundary. inv_n is 1.0 / n. Mean squares outside the range
// where the single-precision seed is safe take the plain expression.
__device__ __forceinline__ float inv_rms(double sum_sq, double inv_n, float eps) {
    const double d = fma(sum_sq, inv_n, (double)eps);
    const float df = (float)d;
    if (!(df > 1e-30f && df < 1e30f)) return (float)(1.0 / sqrt(d));
    double r = (double)rsqrtf(df);
    const double h = -0.5 * d;
    r = r * fma(h * r, r, 1.5);
    r = r * fma(h * r, r, 1.5);
    return (float)r;
}

}  // namespace b200

#endif  // B200_COMMON_CUH
