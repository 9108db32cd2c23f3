// hip/hip_fp16.h -- HOST stand-in (see hip_runtime.h in this folder): the fp16 storage type and the conversions the
// reference's device code uses, round to nearest even, subnormals kept. Test infrastructure only.
#ifndef SIMT_EMUL_HIP_FP16_H
#define SIMT_EMUL_HIP_FP16_H

#include "hip_runtime.h"

#ifdef __cplusplus
struct __half {
    uint16_t x;
    __half() = default;
    __half(float f);                 // (__half)value, rounding to nearest even
    operator float() const;          // (float)h
};

inline __half __float2half(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t a = u & 0x7fffffffu;
    __half h;
    if (a >= 0x7f800000u) {                       // inf / nan
        h.x = (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u : 0u));
    } else if (a >= 0x477ff000u) {                // rounds to >= 65520: inf
        h.x = (uint16_t)(sign | 0x7c00u);
    } else if (a >= 0x38800000u) {                // normal half
        const uint32_t m = a - 0x38000000u;       // rebias the exponent (127 - 15) << 23
        const uint32_t r = m + 0xfffu + ((m >> 13) & 1u);
        h.x = (uint16_t)(sign | (r >> 13));
    } else if (a >= 0x33000000u) {                // subnormal half: value * 2^24 rounded to an integer
        const int e = (int)(a >> 23);             // 102 .. 112
        const uint32_t man = (a & 0x7fffffu) | 0x800000u;
        const int shift = 126 - e;                // 14 .. 24 bits to drop
        const uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
        h.x = (uint16_t)(sign | (q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u)));
    } else {
        h.x = (uint16_t)sign;
    }
    return h;
}
inline __half __float2half_rn(float f) { return __float2half(f); }

inline float __half2float(__half h) {
    const uint32_t sign = (uint32_t)(h.x & 0x8000u) << 16, e = (h.x >> 10) & 31u, m = h.x & 0x3ffu;
    uint32_t u;
    if (e == 31u) u = sign | 0x7f800000u | (m << 13);
    else if (e != 0u) u = sign | ((e + 112u) << 23) | (m << 13);
    else if (m == 0u) u = sign;
    else {
        int k = 0;
        uint32_t mm = m;
        while (!(mm & 0x400u)) { mm <<= 1; ++k; }
        u = sign | ((uint32_t)(113 - k) << 23) | ((mm & 0x3ffu) << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}
// two halves; the packed operations round each result once to fp16 (a product of two halves is exact in fp32; a
// difference is exact there unless the exponents are more than 13 apart)
struct alignas(4) __half2 { __half x, y; };
inline __half2 __half2half2(__half h) { return __half2{h, h}; }
inline __half2 __float2half2_rn(float f) { return __half2{__float2half(f), __float2half(f)}; }
inline __half2 __floats2half2_rn(float a, float b) { return __half2{__float2half(a), __float2half(b)}; }
inline float2 __half22float2(__half2 h) { return float2{__half2float(h.x), __half2float(h.y)}; }
inline __half2 __hmul2(__half2 a, __half2 b) {
    return __half2{__float2half(__half2float(a.x) * __half2float(b.x)), __float2half(__half2float(a.y) * __half2float(b.y))};
}
inline __half2 __hsub2(__half2 a, __half2 b) {
    return __half2{__float2half(__half2float(a.x) - __half2float(b.x)), __float2half(__half2float(a.y) - __half2float(b.y))};
}
inline __half2 __hadd2(__half2 a, __half2 b) {
    return __half2{__float2half(__half2float(a.x) + __half2float(b.x)), __float2half(__half2float(a.y) + __half2float(b.y))};
}
inline __half::__half(float f) : x(__float2half(f).x) {}
inline __half::operator float() const { return __half2float(*this); }
inline uint16_t __half_as_ushort(__half h) { return h.x; }
inline __half __ushort_as_half(uint16_t x) { __half h; h.x = x; return h; }
#endif

#endif  // SIMT_EMUL_HIP_FP16_H
