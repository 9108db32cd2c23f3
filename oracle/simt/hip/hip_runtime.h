// hip/hip_runtime.h -- HOST stand-in for the HIP runtime header, for running the reference's own device code
// (src/gpu_ops.hip with src/q8_device.h) and its own launchers (src/gpu_ops.cpp) on the CPU. TEST INFRASTRUCTURE ONLY:
// it exists so that the checkers under oracle/ can be pinned against the reference's kernels themselves, which have
// no CPU counterpart; nothing in the product includes or links it.
//
// Execution model: a kernel launch runs its blocks one after the other; the threads of a block are real host threads
// (one std::thread per GPU thread), so __syncthreads is a barrier over the block, a wave is 32 consecutive threads with
// a barrier of its own, and __shfl_xor / __shfl_up / __shfl_down exchange values through the wave's slot array between
// two waits on that barrier. As on the GPU, every thread of a wave must reach a shuffle and every thread of a block
// must reach a __syncthreads. __shared__ variables are function-local statics (one block runs at a time). Arithmetic
// is the host's IEEE fp32 (compile with -ffp-contract=off); the fast-math intrinsics map to the libm functions.
#ifndef SIMT_EMUL_HIP_RUNTIME_H
#define SIMT_EMUL_HIP_RUNTIME_H

#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef __cplusplus
#include <algorithm>
#include <barrier>
#include <memory>

// ------------------------------------------------------------------ host API types (what src/gpu_ops.cpp uses)
typedef int hipError_t;
enum { hipSuccess = 0, hipErrorInvalidValue = 1, hipErrorInvalidDeviceFunction = 98 };
typedef struct simt_stream* hipStream_t;
typedef struct simt_module* hipModule_t;
typedef struct simt_function* hipFunction_t;

extern "C" {
hipError_t hipModuleGetFunction(hipFunction_t* fn, hipModule_t mod, const char* name);
hipError_t hipModuleUnload(hipModule_t mod);
hipError_t hipModuleLaunchKernel(hipFunction_t fn, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                                 unsigned bz, unsigned shared_bytes, hipStream_t stream, void** args, void** extra);
const char* hipGetErrorString(hipError_t e);
}

// ------------------------------------------------------------------ device-side vocabulary
struct simt_dim3 { unsigned x, y, z; };
struct simt_wave {
    std::barrier<> bar;
    unsigned long long slot[32];
    int n;
    explicit simt_wave(int threads) : bar(threads), n(threads) {}
};
struct simt_ctx {           // per emulated thread
    simt_dim3 tid, bid;
    std::barrier<>* block;
    simt_wave* wave;
    int lane;
};
extern thread_local simt_ctx simt_self;
extern simt_dim3 simt_block_dim, simt_grid_dim;

#define threadIdx (simt_self.tid)
#define blockIdx (simt_self.bid)
#define blockDim (simt_block_dim)
#define gridDim (simt_grid_dim)

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __shared__ static
#define __launch_bounds__(...)
#define __restrict__

struct alignas(8) float2 { float x, y; };
struct alignas(16) float4 { float x, y, z, w; };
struct alignas(8) int2 { int x, y; };
struct alignas(16) int4 { int x, y, z, w; };
struct alignas(16) uint4 { unsigned x, y, z, w; };
struct alignas(8) uint2 { unsigned x, y; };
inline uint4 make_uint4(unsigned x, unsigned y, unsigned z, unsigned w) { return uint4{x, y, z, w}; }
inline uint2 make_uint2(unsigned x, unsigned y) { return uint2{x, y}; }
inline int4 make_int4(int x, int y, int z, int w) { return int4{x, y, z, w}; }
inline float4 make_float4(float x, float y, float z, float w) { return float4{x, y, z, w}; }
inline float2 make_float2(float x, float y) { return float2{x, y}; }

inline void __syncthreads() { simt_self.block->arrive_and_wait(); }

template <typename T>
inline T simt_exchange(T v, int src_lane) {
    static_assert(sizeof(T) <= 8, "shuffles carry at most 8 bytes");
    simt_wave& w = *simt_self.wave;
    unsigned long long bits = 0;
    memcpy(&bits, &v, sizeof(T));
    w.slot[simt_self.lane] = bits;
    w.bar.arrive_and_wait();
    T r = v;
    if (src_lane >= 0 && src_lane < w.n) memcpy(&r, &w.slot[src_lane], sizeof(T));
    w.bar.arrive_and_wait();
    return r;
}
template <typename T>
inline T __shfl_xor(T v, int mask, int width = 32) {
    const int l = simt_self.lane, s = l ^ mask;
    return simt_exchange(v, (s / width == l / width) ? s : l);
}
// (the *_sync spellings take a lane mask first: every lane of the wave takes part here)
template <typename T>
inline T __shfl_xor_sync(unsigned long long, T v, int mask, int width = 32) { return __shfl_xor(v, mask, width); }
template <typename T>
inline T __shfl_up(T v, unsigned delta, int width = 32) {
    const int l = simt_self.lane, s = l - (int)delta;
    return simt_exchange(v, (s >= 0 && s / width == l / width) ? s : l);
}
template <typename T>
inline T __shfl_down(T v, unsigned delta, int width = 32) {
    const int l = simt_self.lane, s = l + (int)delta;
    return simt_exchange(v, (s / width == l / width) ? s : l);
}
template <typename T>
inline T __shfl(T v, int src, int width = 32) {
    const int l = simt_self.lane;
    return simt_exchange(v, l / width * width + (src % width));
}

// mask of the wave's lanes whose predicate holds
inline unsigned long long __ballot(int pred) {
    simt_wave& w = *simt_self.wave;
    w.slot[simt_self.lane] = pred ? 1ull : 0ull;
    w.bar.arrive_and_wait();
    unsigned long long m = 0;
    for (int l = 0; l < w.n; ++l) m |= w.slot[l] << l;
    w.bar.arrive_and_wait();
    return m;
}
// DPP row_xmask (control 0x160 | M): the value of the lane whose index differs in bits M inside its row of 16
inline int simt_mov_dpp(int v, int ctrl) {
    return simt_exchange(v, (ctrl & 0x1f0) == 0x160 ? (simt_self.lane ^ (ctrl & 15)) : simt_self.lane);
}
#define __builtin_amdgcn_mov_dpp(v, ctrl, row_mask, bank_mask, bound_ctrl) simt_mov_dpp((v), (ctrl))
// V_PERM_B32: byte i of the result is byte sel_i of the 8 bytes {hi, lo} (0-3: lo, 4-7: hi; 12: 0x00; >= 13: 0xff)
inline uint32_t simt_perm(uint32_t hi, uint32_t lo, uint32_t sel) {
    const unsigned long long both = ((unsigned long long)hi << 32) | lo;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const unsigned s = (sel >> (8 * i)) & 0xffu;
        unsigned b = 0;
        if (s < 8) b = (unsigned)(both >> (8 * s)) & 0xffu;
        else if (s < 12) b = ((both >> (16 * (s - 8) + 15)) & 1u) ? 0xffu : 0u;   // sign of a 16-bit half
        else if (s == 12) b = 0;
        else b = 0xffu;
        r |= b << (8 * i);
    }
    return r;
}
#define __builtin_amdgcn_perm(hi, lo, sel) simt_perm((hi), (lo), (sel))
// the matrix instruction is outside what these checkers run: it compiles, and stops the program if reached
template <typename A, typename Cc>
inline Cc simt_wmma_unavailable(A, A, Cc c) { __builtin_trap(); return c; }
#define __builtin_amdgcn_wmma_f32_16x16x16_f16_w32(a, b, c) simt_wmma_unavailable((a), (b), (c))

inline int atomicAdd(int* p, int v) { return __atomic_fetch_add(p, v, __ATOMIC_RELAXED); }
inline unsigned atomicAdd(unsigned* p, unsigned v) { return __atomic_fetch_add(p, v, __ATOMIC_RELAXED); }
inline int atomicMin(int* p, int v) {
    int old = __atomic_load_n(p, __ATOMIC_RELAXED);
    while (v < old && !__atomic_compare_exchange_n(p, &old, v, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) {}
    return old;
}
inline int atomicMax(int* p, int v) {
    int old = __atomic_load_n(p, __ATOMIC_RELAXED);
    while (v > old && !__atomic_compare_exchange_n(p, &old, v, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) {}
    return old;
}

inline float __fmul_rn(float a, float b) { return a * b; }
inline float __fadd_rn(float a, float b) { return a + b; }
inline float __fsub_rn(float a, float b) { return a - b; }
inline float __fdiv_rn(float a, float b) { return a / b; }
inline float __expf(float x) { return expf(x); }
inline float __logf(float x) { return logf(x); }
inline float __powf(float x, float y) { return powf(x, y); }
inline float __frcp_rn(float x) { return 1.0f / x; }
inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
inline uint32_t __float_as_uint(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
inline int __float_as_int(float f) { int u; memcpy(&u, &f, 4); return u; }
inline float __uint_as_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
inline float __int_as_float(int u) { float f; memcpy(&f, &u, 4); return f; }
inline int min(int a, int b) { return a < b ? a : b; }
inline int max(int a, int b) { return a > b ? a : b; }
inline unsigned min(unsigned a, unsigned b) { return a < b ? a : b; }
inline unsigned max(unsigned a, unsigned b) { return a > b ? a : b; }
inline long long min(long long a, long long b) { return a < b ? a : b; }
inline long long max(long long a, long long b) { return a > b ? a : b; }
inline float min(float a, float b) { return fminf(a, b); }
inline float max(float a, float b) { return fmaxf(a, b); }

// ------------------------------------------------------------------ kernel registry (name -> typed launch)
typedef void (*simt_thunk)(void** args);
void simt_register(const char* name, simt_thunk run_one_thread);

template <typename... A, size_t... I>
inline void simt_call(void (*k)(A...), void** args, std::index_sequence<I...>) {
    k(*reinterpret_cast<std::remove_reference_t<A>*>(args[I])...);
}
// SIMT_KERNEL(name): makes the kernel `name` (a plain function here) launchable by that name
#define SIMT_KERNEL(name)                                                                                    \
    namespace {                                                                                              \
    template <typename... A>                                                                                 \
    void simt_thunk_of_##name(void (*k)(A...), void** args) { simt_call(k, args, std::index_sequence_for<A...>{}); } \
    struct simt_reg_##name {                                                                                 \
        simt_reg_##name() { simt_register(#name, [](void** args) { simt_thunk_of_##name(&name, args); }); }   \
    } simt_reg_instance_##name;                                                                              \
    }

#endif  // __cplusplus
#endif  // SIMT_EMUL_HIP_RUNTIME_H
