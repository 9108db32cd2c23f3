// layer_ops.cu -- host launchers and the C ABI of libb200_layer_ops.so (include/b200_layer_ops.h). Argument checks
// and error codes follow the reference's launchers (src/gpu_ops.cpp:66-86); the launch shapes are B200's own: the
// kernel variant and the threads per row are chosen from the row width and storage type only, the grid from the row
// count and the SM count.

#include "b200_layer_ops.h"

#include <limits.h>
#include <math.h>
#include <string.h>

#include <atomic>
#include <cmath>
#include <mutex>
#include <stdlib.h>
#include <type_traits>

#include "embed.cuh"
#include "internal.h"
#include "kv_store.cuh"
#include "moe_group.cuh"
#include "moe_router.cuh"
#include "norm_chains.cuh"
#include "q8_side.cuh"
#include "qk_norm_rope.cuh"
#include "rmsnorm.cuh"
#include "rope_f16.cuh"
#include "stream_ops.cuh"
#include "swiglu.cuh"
#include "window_ops.cuh"

using namespace b200;

namespace {

std::atomic<bool> g_ready{false};
std::atomic<unsigned long long> g_launches{0};

}  // namespace

namespace b200 {

bool lib_ready() { return g_ready.load(std::memory_order_acquire); }

cudaError_t launched() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

}  // namespace b200

namespace {

// SM count of the current device, cached per device (atomics: launchers run on any thread)
int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }
inline int round_up(int v, int m) { return (v + m - 1) / m * m; }


// Resident CTAs of `block` threads a B200 SM holds when only the thread count limits it
inline long long resident_ctas(int block) { return (long long)sm_count() * (2048 / block > 0 ? 2048 / block : 1); }

// CTAs of this kernel that are resident on the whole device at once (registers and shared memory counted): the grid
// of a kernel whose CTAs walk their rows with a grid stride, so that no CTA waits for another to retire. Cached per
// kernel and launch shape (the occupancy query costs microseconds).
template <typename K>
long long persistent_grid(K kernel, int block, size_t smem) {
    struct Entry { const void* f; int block; size_t smem; int dev; int per_sm; };
    thread_local Entry cache[16];
    thread_local int used = 0;
    int dev = 0;
    (void)cudaGetDevice(&dev);
    const void* f = reinterpret_cast<const void*>(kernel);
    for (int i = 0; i < used; ++i)
        if (cache[i].f == f && cache[i].block == block && cache[i].smem == smem && cache[i].dev == dev)
            return (long long)cache[i].per_sm * sm_count();
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, smem) != cudaSuccess || per_sm < 1) {
        (void)cudaGetLastError();
        per_sm = 1;
    }
    cache[used % 16] = {f, block, smem, dev, per_sm};
    if (used < 16) ++used;
    return (long long)per_sm * sm_count();
}

// Launch with programmatic stream serialisation allowed: the kernels launched this way start with pdl_entry(), so
// they may be scheduled while the kernel before them in the stream drains (see common.cuh). A failed launch leaves its
// error for launched() to return.
template <typename... KA, typename... A>
inline void launch_pdl(void (*kernel)(KA...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KA>(args)...);
}

// ---------------------------------------------------------------- residual add + RMSNorm

// How a row of nvec 16-byte vectors is spread over threads. A function of the row alone: the summation order of a
// row must not depend on the batch.
struct NormPlan {
    bool cta_row;
    int tpr, vpt;
};

bool plan_norm(int nvec, NormPlan* p) {
    if (nvec <= 64) { *p = {false, next_pow2((nvec + 1) / 2), 2}; return true; }
    // four vectors per thread when that fills whole warps (64 bytes of a row in flight per thread), else two
    int vpt = nvec % 128 == 0 ? 4 : 2;
    if (nvec == 128) { *p = {true, 32, 4}; return true; }
    int tpr = round_up((nvec + vpt - 1) / vpt, 32);
    while (tpr > 1024 && vpt < 8) { vpt *= 2; tpr = round_up((nvec + vpt - 1) / vpt, 32); }
    if (tpr > 1024) return false;
    *p = {true, tpr, vpt};
    return true;
}

template <typename IO, typename WT, int VPT>
cudaError_t launch_norm_vec(const NormPlan& p, const IO* x_in, const IO* add, IO* x_out, const WT* w, IO* y, int n,
                            long long T, float eps, cudaStream_t stream) {
    if (p.cta_row) {
        const long long res = persistent_grid(k_add_rmsnorm<IO, WT, VPT, true>, p.tpr, 0);
        const long long grid = T < res ? T : res;
        launch_pdl((k_add_rmsnorm<IO, WT, VPT, true>), (unsigned)grid, p.tpr, 0, stream, x_in, add, x_out, w, y, n, T, eps, p.tpr);
    } else {
        // several rows per CTA; with few rows, fewer per CTA so that the rows spread over the SMs
        int rows = 256 / p.tpr;
        while (rows > 1 && rows * p.tpr > 32 && (T + rows - 1) / rows < 2LL * sm_count()) rows >>= 1;
        const int block = rows * p.tpr < 32 ? 32 : rows * p.tpr;
        const int rpp = block / p.tpr;
        long long grid = (T + rpp - 1) / rpp;
        const long long res = persistent_grid(k_add_rmsnorm<IO, WT, VPT, false>, block, 0);
        if (grid > res) grid = res;
        launch_pdl((k_add_rmsnorm<IO, WT, VPT, false>), (unsigned)grid, block, 0, stream, x_in, add, x_out, w, y, n, T, eps, p.tpr);
    }
    return launched();
}

// side (fp32 rows): the activation side outputs of y (src/q8_device.h:54-104). Where the row shape takes the trimmed
// kernel, the kernel writes them itself from the registers that hold y: the 16-bit copy when side->xh is set (8-byte
// aligned), the int8 formats when side->qK is set (n % 256 == 0, q0 / qK 4-byte aligned). *xh_done / *q8_done say
// what was written; the caller runs the side kernel over y for the rest.
template <typename IO, typename WT>
cudaError_t launch_add_rmsnorm(const IO* x_in, const IO* add, IO* x_out, const WT* w, IO* y, int n, long long T,
                               float eps, cudaStream_t stream, const Q8Side* side = nullptr, bool* xh_done = nullptr,
                               bool* q8_done = nullptr) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n <= 0 || !x_in || !y || (add && (!x_out || x_out == x_in))) return cudaErrorInvalidValue;
    constexpr int VE = Io<IO>::VE;
    NormPlan p;
    const bool vec = n % VE == 0 && al16(x_in) && al16(y) && (!add || (al16(add) && al16(x_out))) &&
                     (!w || al16(w)) && plan_norm(n / VE, &p);
    if constexpr (std::is_same<WT, float>::value && !std::is_same<IO, __half>::value) {
        // exact fit of whole warps with gammas: the trimmed kernel
        if (vec && p.cta_row && w && p.tpr <= 512 && (n / VE) == p.tpr * p.vpt && (p.vpt == 2 || p.vpt == 4)) {
// The residual variant runs one CTA per row (it has no loads in flight across rows, and CTAs that retire and are
// replaced in row order keep the rows being read and written next to each other in memory: 1.04 of the copy bandwidth
// on 262,144 rows of 5120 against 0.96 with a grid of resident CTAs walking strided rows); on narrow rows (two vectors
// per thread) a CTA takes four consecutive rows and fetches the next while it reduces the current one (16,384 rows of
// 2560: 0.86 against 0.75). The plain norm keeps the resident grid, whose CTAs fetch their next row while they reduce
// the current one (0.97 against 0.76).
#define NORM_FAST3(V, A, M, XHV, Q8V, SIDE)                                                          \
    do {                                                                                             \
        const int rpc = (A) ? ((V) <= 2 ? 4 : 1) : ((Q8V) ? 4 : 0);   /* (int8 side outputs: 0.78 against 0.73) */ \
        long long grid = rpc ? (T + rpc - 1) / rpc : persistent_grid(k_add_rmsnorm_fast<IO, V, A, M, XHV, Q8V>, p.tpr, 0); \
        if (grid > T) grid = T;                                                                      \
        if (grid > INT_MAX) return cudaErrorInvalidValue;                                            \
        launch_pdl((k_add_rmsnorm_fast<IO, V, A, M, XHV, Q8V>), (unsigned)grid, p.tpr, 0, stream, x_in, add, x_out, w, y, n, T, eps, SIDE, rpc); \
    } while (0)
#define NORM_FAST2(V, A, XHV, Q8V, SIDE)                                                             \
    do {                                                                                             \
        if (p.tpr <= 160) NORM_FAST3(V, A, 160, XHV, Q8V, SIDE);                                     \
        else if (p.tpr <= 320) NORM_FAST3(V, A, 320, XHV, Q8V, SIDE);                                \
        else NORM_FAST3(V, A, 512, XHV, Q8V, SIDE);                                                  \
    } while (0)
#define NORM_FAST(XHV, Q8V, SIDE)                                                                    \
    do {                                                                                             \
        if (p.vpt == 4) { if (add) NORM_FAST2(4, true, XHV, Q8V, SIDE); else NORM_FAST2(4, false, XHV, Q8V, SIDE); } \
        else { if (add) NORM_FAST2(2, true, XHV, Q8V, SIDE); else NORM_FAST2(2, false, XHV, Q8V, SIDE); }            \
    } while (0)
            if constexpr (std::is_same<IO, float>::value) {
                const bool do_xh = side && side->xh && (reinterpret_cast<uintptr_t>(side->xh) & 7) == 0;
                const bool do_q8 = side && side->qK && n % 256 == 0 && n <= 8192 &&
                                   ((reinterpret_cast<uintptr_t>(side->q0) | reinterpret_cast<uintptr_t>(side->qK)) & 3) == 0;
                if (do_xh || do_q8) {
                    if (do_xh && do_q8) NORM_FAST(true, true, *side);
                    else if (do_q8) NORM_FAST(false, true, *side);
                    else NORM_FAST(true, false, *side);
                    if (xh_done) *xh_done = do_xh;
                    if (q8_done) *q8_done = do_q8;
                    return launched();
                }
            }
            NORM_FAST(false, false, Q8Side{});
#undef NORM_FAST3
#undef NORM_FAST2
#undef NORM_FAST
            return launched();
        }
    }
    if (!vec) {
        const long long cap = resident_ctas(256);
        k_add_rmsnorm_generic<IO, WT><<<(unsigned)(T < cap ? T : cap), 256, 0, stream>>>(x_in, add, x_out, w, y, n, T, eps);
        return launched();
    }
    switch (p.vpt) {
        case 2: return launch_norm_vec<IO, WT, 2>(p, x_in, add, x_out, w, y, n, T, eps, stream);
        case 4: return launch_norm_vec<IO, WT, 4>(p, x_in, add, x_out, w, y, n, T, eps, stream);
        default: return launch_norm_vec<IO, WT, 8>(p, x_in, add, x_out, w, y, n, T, eps, stream);
    }
}

inline Q8Side side_of(const qmatvec_q8* q8) {
    return Q8Side{q8->q0, q8->d0, q8->qK, q8->dK, q8->bsK, q8->s0, q8->xh, q8->xh_bf16};
}

cudaError_t launch_q8_side(const float* x, long long K, const qmatvec_q8* q8, cudaStream_t stream) {
    if (!q8->qK && !q8->xh) return cudaSuccess;  // nothing wanted (src/q8_device.h:35)
    Q8Side o = side_of(q8);
    const long long nblk = (K + 255) / 256, cap = resident_ctas(256) * 8;
    long long grid = (nblk + 7) / 8;   // a warp per block, 8 warps per CTA
    if (grid > cap) grid = cap;
    const bool vec = al16(x) && (!o.xh || al16(o.xh)) && (!o.qK || ((reinterpret_cast<uintptr_t>(o.q0) | reinterpret_cast<uintptr_t>(o.qK)) & 7) == 0);
    if (vec) k_q8_side<true><<<(unsigned)grid, 256, 0, stream>>>(x, K, o);
    else k_q8_side<false><<<(unsigned)grid, 256, 0, stream>>>(x, K, o);
    return launched();
}

// ---------------------------------------------------------------- SwiGLU

// side (fp32): as for launch_add_rmsnorm. The int8 formats are fused when n % 32 == 0 and q0 / qK are 4-byte aligned.
template <typename IO, bool FAST>
cudaError_t launch_swiglu(const IO* g, const IO* u, IO* out, long long n, cudaStream_t stream, const Q8Side* side = nullptr,
                          bool* xh_done = nullptr, bool* q8_done = nullptr) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (n < 0 || (n > 0 && (!g || !u || !out))) return cudaErrorInvalidValue;
    if (n == 0) return cudaSuccess;
    constexpr int VE = Io<IO>::VE, UNROLL = 4;
    if (al16(g) && al16(u) && al16(out)) {
        const long long nvec = n / VE, per_cta = 256LL * UNROLL;
        long long grid = (nvec + per_cta - 1) / per_cta;
        // one tile per CTA: CTAs that retire and are replaced in tile order keep the tiles in flight next to each other
        // in memory (1.07 of the copy bandwidth on the 27B-shape FFN rows against 1.01 with a capped grid walking tiles)
        const long long cap = INT_MAX;
        if (grid > cap) grid = cap;
        if (grid < 1) grid = 1;
        if constexpr (std::is_same<IO, float>::value) {
            const bool do_xh = side && side->xh && n % VE == 0 && (reinterpret_cast<uintptr_t>(side->xh) & 7) == 0;
            const bool do_q8 = side && side->qK && n % 32 == 0 &&
                               ((reinterpret_cast<uintptr_t>(side->q0) | reinterpret_cast<uintptr_t>(side->qK)) & 3) == 0;
            if (do_q8) {
                if (do_xh) launch_pdl((k_swiglu_q8<UNROLL, true>), (unsigned)grid, 256, 0, stream, g, u, out, n, *side);
                else launch_pdl((k_swiglu_q8<UNROLL, false>), (unsigned)grid, 256, 0, stream, g, u, out, n, *side);
                if (xh_done) *xh_done = do_xh;
                if (q8_done) *q8_done = true;
                return launched();
            }
            if (do_xh) {
                launch_pdl((k_swiglu<IO, FAST, UNROLL, true>), (unsigned)grid, 256, 0, stream, g, u, out, n, side->xh, side->xh_bf16);
                if (xh_done) *xh_done = true;
                return launched();
            }
        }
        launch_pdl((k_swiglu<IO, FAST, UNROLL>), (unsigned)grid, 256, 0, stream, g, u, out, n, nullptr, 0);
    } else {
        const long long cap = resident_ctas(256) * 8;
        long long grid = (n + 255) / 256;
        if (grid > cap) grid = cap;
        k_swiglu_scalar<IO, FAST><<<(unsigned)grid, 256, 0, stream>>>(g, u, out, n);
    }
    return launched();
}

template <typename IO, bool FAST>
cudaError_t launch_swiglu_rows(const IO* gate, const IO* up, IO* out, long long rows, int h, long long gs, long long us,
                               cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (rows < 0 || h <= 0 || !gate || !up || !out || gs < 0 || us < 0) return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    constexpr int VE = Io<IO>::VE;
    const bool vec = h % VE == 0 && gs % VE == 0 && us % VE == 0 && al16(gate) && al16(up) && al16(out);
    const long long work = vec ? rows * (h / VE) : rows * (long long)h;
    const long long cap = INT_MAX;   // one step per thread, CTAs in row order (as launch_swiglu)
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_swiglu_strided_vec<IO, FAST><<<(unsigned)grid, 256, 0, stream>>>(gate, up, out, rows, h, gs, us);
    else k_swiglu_strided<IO, FAST><<<(unsigned)grid, 256, 0, stream>>>(gate, up, out, rows, h, gs, us);
    return launched();
}

// ---------------------------------------------------------------- q/k norm + RoPE

// Stand-in for a missing gamma in the vector kernel (multiplying by 1.0f leaves every bit alone)
__device__ float g_ones[1024];
bool g_ones_ready[64];
std::mutex g_ones_lock;   // first use on a device may come from several threads at once

const float* ones_vector() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_ones) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> hold(g_ones_lock);
    if (!g_ones_ready[dev]) {
        float h[1024];
        for (int i = 0; i < 1024; ++i) h[i] = 1.0f;
        if (cudaMemcpy(p, h, sizeof(h), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
        g_ones_ready[dev] = true;
    }
    return p;
}

// inv_freq[i] = freq_base^(-2 i / n_rot) by the CPU reference's own expression (src/qwen_ops.cpp:18), so that
// pos * inv_freq[i] is the reference's angle to the last bit. Kept per thread for the last (base, n_rot) seen.
const RopeFreq& rope_freq(float freq_base, int n_rot) {
    thread_local RopeFreq fr;
    thread_local float base = -1.0f;
    thread_local int rot = -1;
    if (base != freq_base || rot != n_rot) {
        for (int i = 0; i < n_rot / 2; ++i) fr.inv_freq[i] = std::pow((double)freq_base, -2.0 * i / n_rot);
        for (int i = n_rot / 2; i < B200_MAX_ROT_PAIRS; ++i) fr.inv_freq[i] = 0.0;
        base = freq_base;
        rot = n_rot;
    }
    return fr;
}

struct KvTarget {   // where the K heads go when they are written into the KV cache instead of k_out
    __half* cache;
    int kv_stride, kv_shift;
    long long kv_bstride;
};

// Tables of a call whose cos / sin were computed beforehand (gpu_rope_table): [T][n_rot / 2] fp32 each
struct RopeTables {
    const float* cos_tab;
    const float* sin_tab;
};

cudaError_t launch_rope_table(const int* positions, int pos0, long long T, int n_rot, int rot_pairs, float freq_base,
                              const float* ff, float* cos_out, float* sin_out, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n_rot < 0 || n_rot % 2 != 0 || n_rot / 2 > B200_MAX_ROT_PAIRS || rot_pairs > n_rot / 2 ||
        (!positions && pos0 < 0) || (n_rot > 0 && (!cos_out || !sin_out)))
        return cudaErrorInvalidValue;
    if (n_rot == 0) return cudaSuccess;   // no rotation: no table
    const int half = n_rot / 2;
    if (rot_pairs <= 0) rot_pairs = half;
    const RopeFreq& fr = rope_freq(freq_base, n_rot);
    const bool fast = !ff && freq_base >= 1.0f;   // every angle below 2^31: the range of the kernel's own sincos
    const bool vec = half % 4 == 0 && al16(cos_out) && al16(sin_out);
    const int tpp = 256 / (half / (vec ? 4 : 1));
    long long grid = (T + tpp - 1) / tpp;
    const long long cap = resident_ctas(256) * 4;
    if (grid > cap) grid = cap;
#define ROPE_TAB(F, P) launch_pdl((k_rope_table<F, P>), (unsigned)grid, 256, 0, stream, positions, pos0, T, half, rot_pairs, ff, cos_out, sin_out, fr)
    if (fast) { if (vec) ROPE_TAB(true, 4); else ROPE_TAB(true, 1); }
    else { if (vec) ROPE_TAB(false, 4); else ROPE_TAB(false, 1); }
#undef ROPE_TAB
    return launched();
}

template <typename IO, bool KVC = false>
cudaError_t launch_qk(const IO* qfull, const IO* k, const float* q_norm, const float* k_norm, IO* q_out, IO* k_out,
                      int n_q, int n_kv, int D, int n_rot, int rot_pairs, const int* positions, int pos0, long long T,
                      float freq_base, float eps, int gated, int qk_norm, const float* ff, cudaStream_t stream,
                      KvTarget kv = KvTarget{nullptr, 0, 0, 0}, const RopeTables* tabs = nullptr) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (tabs && n_rot > 0 && (!tabs->cos_tab || !tabs->sin_tab)) return cudaErrorInvalidValue;
    if (KVC) {
        if (!kv.cache || n_kv <= 0 || kv.kv_shift < 0 || kv.kv_shift > 30 || kv.kv_stride < n_kv * D || kv.kv_bstride < 0)
            return cudaErrorInvalidValue;
        k_out = const_cast<IO*>(k);   // unused; keeps the pointer checks below uniform
    }
    // the checks of attention_forward_opts (src/attention.cpp:139-143) that concern this step
    if (T <= 0 || n_q < 0 || n_kv < 0 || n_q + n_kv <= 0 || D <= 0 || D > 1024 || n_rot < 0 || n_rot > D ||
        n_rot % 2 != 0 || n_rot / 2 > B200_MAX_ROT_PAIRS || rot_pairs > n_rot / 2 || (!positions && pos0 < 0) ||
        (n_q > 0 && (!qfull || !q_out)) || (n_kv > 0 && (!k || !k_out)) || (gated && q_out == qfull))
        return cudaErrorInvalidValue;
    if (rot_pairs <= 0) rot_pairs = n_rot / 2;
    QkArgs a;
    a.qfull = qfull; a.k = k; a.q_out = q_out; a.k_out = k_out;
    a.q_norm = q_norm; a.k_norm = k_norm; a.ff = ff; a.positions = positions;
    a.n_q = n_q; a.n_kv = n_kv; a.D = D; a.q_stride = gated ? 2 * D : D;
    a.n_rot = n_rot; a.rot_pairs = rot_pairs; a.pos0 = pos0; a.do_norm = qk_norm ? 1 : 0;
    a.T = T; a.eps = eps;
    a.k_cache = KVC ? kv.cache : nullptr; a.kv_stride = kv.kv_stride; a.kv_shift = kv.kv_shift; a.kv_bstride = kv.kv_bstride;
    const bool tab = tabs && n_rot > 0;
    a.cos_tab = tab ? tabs->cos_tab : nullptr;
    a.sin_tab = tab ? tabs->sin_tab : nullptr;
    static const RopeFreq no_freq = {};   // the kernels that read tables take no multipliers
    const RopeFreq& fr = tab ? no_freq : rope_freq(freq_base, n_rot);

    constexpr int VE = Io<IO>::VE;
    const int NV = D / VE;
    int ppt = 0;
    if (D % VE == 0 && n_rot % (2 * VE) == 0 && (n_q == 0 || (al16(qfull) && al16(q_out))) &&
        (n_kv == 0 || (al16(k) && al16(k_out))) && (!q_norm || al16(q_norm)) && (!k_norm || al16(k_norm)) &&
        (!KVC || (al16(kv.cache) && kv.kv_stride % 8 == 0 && kv.kv_bstride % 8 == 0))) {
        for (int c = 1; c <= 2 && !ppt; ++c)
            if (NV % (2 * c) == 0) {
                const int tph = NV / (2 * c);
                if (tph <= 32 && (tph & (tph - 1)) == 0) ppt = c;
            }
    }
    if (!ppt) {
        const long long cap = resident_ctas(128);
        k_qk_norm_rope_generic<IO><<<(unsigned)(T < cap ? T : cap), 128, 0, stream>>>(a, fr);
        return launched();
    }
    if (qk_norm && (!q_norm || !k_norm)) {
        const float* ones = ones_vector();
        if (!ones) return cudaErrorInvalidDeviceFunction;
        if (!q_norm) a.q_norm = ones;
        if (!k_norm) a.k_norm = ones;
    }
    const int tph = NV / (2 * ppt);
    int block = round_up((n_q + n_kv) * tph, 32);
    // The trimmed kernel: one head chunk of exactly block threads, long batches, normalisation on, n_rot / 2 a
    // multiple of 4 floats (16-byte table reads). It takes the whole tiles of 4 tokens; the 0..3 tokens left over go
    // through the general kernel below (a row's bits do not depend on which of the two processed it).
    constexpr int FTT = 4;
    // (no frequency factors and a base >= 1: every angle is then below 2^31, the range of the kernel's own sincos)
    const bool trig_ok = tab ? (al16(a.cos_tab) && al16(a.sin_tab)) : (!ff && freq_base >= 1.0f);
    if (ppt == 1 && qk_norm && trig_ok && (n_q + n_kv) * tph == block && block <= 384 && T >= 8LL * sm_count() && n_rot > 0 &&
        (n_rot / 2) % 4 == 0) {
        const long long tiles = T / FTT;
        const size_t smem = (2 * (size_t)D + 2 * 2 * FTT * (size_t)(n_rot / 2)) * sizeof(float);
        QkArgs m = a;
        m.T = tiles * FTT;
        bool done = false;
        {
            if (tab) {
#define QK_TAB(TTV, FULLV, MINB, DSV, NRV)                                                                            \
    do {                                                                                                              \
        const long long tl = T / TTV;                                                                                 \
        const size_t sm = (2 * (size_t)D + 2 * 2 * TTV * (size_t)(n_rot / 2)) * sizeof(float);                        \
        m.T = tl * TTV;                                                                                               \
        const long long res = persistent_grid(k_qk_norm_rope_fast<IO, TTV, FULLV, KVC, true, MINB, DSV, NRV>, block, sm); \
        launch_pdl((k_qk_norm_rope_fast<IO, TTV, FULLV, KVC, true, MINB, DSV, NRV>), (unsigned)(tl < res ? tl : res), block, sm, stream, m, fr); \
    } while (0)
                if (D == 128 && n_rot == 128) QK_TAB(4, true, 2, 128, 128);         // the heads of the dense configurations
                else if (D == 256 && n_rot == 64) QK_TAB(4, false, 2, 256, 64);    // partial rotary over the first 64 of 256
                else if (n_rot == D) QK_TAB(4, true, 2, 0, 0);
                else QK_TAB(4, false, 2, 0, 0);
#undef QK_TAB
                done = true;
            }
        }
        if (done) {
        } else if (n_rot == D) {
            const long long res = persistent_grid(k_qk_norm_rope_fast<IO, FTT, true, KVC>, block, smem);
            launch_pdl((k_qk_norm_rope_fast<IO, FTT, true, KVC>), (unsigned)(tiles < res ? tiles : res), block, smem, stream, m, fr);
        } else {
            const long long res = persistent_grid(k_qk_norm_rope_fast<IO, FTT, false, KVC>, block, smem);
            launch_pdl((k_qk_norm_rope_fast<IO, FTT, false, KVC>), (unsigned)(tiles < res ? tiles : res), block, smem, stream, m, fr);
        }
        const cudaError_t e = launched();
        const long long rest = T - m.T;
        if (e != cudaSuccess || rest == 0) return e;
        // tail tokens: advance every row pointer and the positions
        const size_t qin = (size_t)n_q * a.q_stride, kin = (size_t)n_kv * D;
        a.qfull = n_q ? static_cast<const IO*>(a.qfull) + m.T * qin : nullptr;
        a.k = n_kv ? static_cast<const IO*>(a.k) + m.T * kin : nullptr;
        a.q_out = n_q ? static_cast<IO*>(a.q_out) + m.T * (size_t)n_q * D : nullptr;
        a.k_out = n_kv ? static_cast<IO*>(a.k_out) + m.T * kin : nullptr;
        if (a.positions) a.positions += m.T;
        else a.pos0 += (int)m.T;
        if (tab) { a.cos_tab += m.T * (size_t)(n_rot / 2); a.sin_tab += m.T * (size_t)(n_rot / 2); }
        a.T = rest;
        T = rest;
    }
    if (block > 384) block = 384 / tph * tph;   // the kernel is built for at most 384 threads, two CTAs per SM
    // tokens per CTA pass: 4 for long batches (64 to 128 bytes of loads in flight per thread), 1 when there are so
    // few tokens that spreading them over the SMs matters more
    const int tt = T >= 8LL * sm_count() ? (ppt == 1 ? 4 : 2) : 1;
    const long long tiles = (T + tt - 1) / tt;
    const size_t smem = 2 * 2 * (size_t)tt * (n_rot / 2 > 0 ? n_rot / 2 : 4) * sizeof(float);
#define QK_LAUNCH(P, TTV)                                                                  \
    do {                                                                                   \
        const long long res = persistent_grid(k_qk_norm_rope<IO, P, TTV, KVC>, block, smem);    \
        launch_pdl((k_qk_norm_rope<IO, P, TTV, KVC>), (unsigned)(tiles < res ? tiles : res), block, smem, stream, a, fr); \
    } while (0)
    if (ppt == 1 && tt == 4) QK_LAUNCH(1, 4);
    else if (ppt == 1) QK_LAUNCH(1, 1);
    else if (tt == 2) QK_LAUNCH(2, 2);
    else QK_LAUNCH(2, 1);
#undef QK_LAUNCH
    return launched();
}

// ---------------------------------------------------------------- embedding gather

template <typename OUT>
cudaError_t launch_embed(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens, OUT* out,
                         int E, long long T, float scale, int* bad_row, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    size_t blk = 0, bb = 0;   // values and bytes per block (src/quant_types.cpp:583-598)
    switch (type) {
        case B200_QT_F32: blk = 1; bb = 4; break;
        case B200_QT_F16: case B200_QT_BF16: blk = 1; bb = 2; break;
        case B200_QT_Q4_0: blk = 32; bb = 18; break;
        case B200_QT_Q4_1: blk = 32; bb = 20; break;
        case B200_QT_Q5_0: blk = 32; bb = 22; break;
        case B200_QT_Q5_1: blk = 32; bb = 24; break;
        case B200_QT_Q8_0: blk = 32; bb = 34; break;
        case B200_QT_Q4_K: blk = 256; bb = 144; break;
        case B200_QT_Q5_K: blk = 256; bb = 176; break;
        case B200_QT_Q6_K: blk = 256; bb = 210; break;
        default: break;
    }
    if (!bb || T <= 0 || E <= 0 || E % 32 != 0 || E % (int)blk != 0 || vocab <= 0 || !table || !tokens || !out || !bad_row ||
        row_bytes < (size_t)E / blk * bb || row_bytes % 2 != 0 || (reinterpret_cast<uintptr_t>(table) & 1u) || !al16(out))
        return cudaErrorInvalidValue;
    const int vec_ok = al16(table) && row_bytes % 16 == 0;
    const long long need = (T + EMBED_WARPS - 1) / EMBED_WARPS;
    const uint8_t* tb = static_cast<const uint8_t*>(table);
#define EMBED(K, TY)                                                                                             \
    do {                                                                                                         \
        const long long res = persistent_grid(K<OUT, TY>, EMBED_WARPS * 32, 0);                                  \
        launch_pdl((K<OUT, TY>), (unsigned)(need < res ? need : res), EMBED_WARPS * 32, 0, stream, tb, row_bytes, vocab, tokens, out, \
                                                                                         E, T, scale, bad_row, vec_ok);     \
    } while (0)
    // Q8_0 / Q4_0 rows of whole 8-block groups in a 16-byte aligned table (every GGUF token_embd of E % 256 == 0).
    // From 8192 tokens on: a warp per slice of a row, one slice per warp, CTAs retiring in slice order, so that what is
    // read and written at any moment lies close together in memory (262,144 rows of 5120, fraction of the copy
    // bandwidth: 1.00 against 0.91 for the whole-row kernel with a resident grid; Q4_0 rows of 2560: 0.93 against 0.84;
    // single cold launches of 32,768 rows of 5120: 0.89 against 0.80 for the kernel below). Shorter batches: a resident
    // grid whose warps keep several slices of a row in flight as bulk copies (2048 rows: 16.7 against 17.8 us).
    if ((type == B200_QT_Q8_0 || type == B200_QT_Q4_0) && vec_ok && E % 256 == 0) {
        if (T < 8192) {
            const long long need_b = (T + EMBED_BULK_WARPS - 1) / EMBED_BULK_WARPS;
#define EMBED_BULK(TY)                                                                                           \
    do {                                                                                                         \
        const long long res = persistent_grid(k_embed_rows_bulk<OUT, TY>, EMBED_BULK_WARPS * 32, 0);             \
        launch_pdl((k_embed_rows_bulk<OUT, TY>), (unsigned)(need_b < res ? need_b : res), EMBED_BULK_WARPS * 32, 0, stream,  \
            tb, row_bytes, vocab, tokens, out, E, T, scale, bad_row);                                             \
    } while (0)
            if (type == B200_QT_Q8_0) EMBED_BULK(B200_QT_Q8_0); else EMBED_BULK(B200_QT_Q4_0);
#undef EMBED_BULK
            return launched();
        }
        const int sb = EMBED_SLICE_BYTES / (type == B200_QT_Q8_0 ? 34 : 18) / 8 * 8;   // blocks per slice, as the kernel's
        const long long slices = T * ((E / 32 + sb - 1) / sb);
        long long grid = (slices + EMBED_WARPS - 1) / EMBED_WARPS;
        if (grid > INT_MAX) grid = INT_MAX;
        if (type == B200_QT_Q8_0)
            launch_pdl((k_embed_rows_sliced<OUT, B200_QT_Q8_0>), (unsigned)grid, EMBED_WARPS * 32, 0, stream, tb, row_bytes, vocab, tokens, out, E, T, scale, bad_row);
        else
            launch_pdl((k_embed_rows_sliced<OUT, B200_QT_Q4_0>), (unsigned)grid, EMBED_WARPS * 32, 0, stream, tb, row_bytes, vocab, tokens, out, E, T, scale, bad_row);
        return launched();
    }
    switch (type) {
        case B200_QT_Q8_0: EMBED(k_embed_rows, B200_QT_Q8_0); break;
        case B200_QT_Q4_0: EMBED(k_embed_rows, B200_QT_Q4_0); break;
        case B200_QT_F32: EMBED(k_embed_rows_any, B200_QT_F32); break;
        case B200_QT_F16: EMBED(k_embed_rows_any, B200_QT_F16); break;
        case B200_QT_BF16: EMBED(k_embed_rows_any, B200_QT_BF16); break;
        case B200_QT_Q4_1: EMBED(k_embed_rows_any, B200_QT_Q4_1); break;
        case B200_QT_Q5_0: EMBED(k_embed_rows_any, B200_QT_Q5_0); break;
        case B200_QT_Q5_1: EMBED(k_embed_rows_any, B200_QT_Q5_1); break;
        case B200_QT_Q4_K: EMBED(k_embed_rows_any, B200_QT_Q4_K); break;
        case B200_QT_Q5_K: EMBED(k_embed_rows_any, B200_QT_Q5_K); break;
        default: EMBED(k_embed_rows_any, B200_QT_Q6_K); break;
    }
#undef EMBED
    return launched();
}

template <typename IO>
cudaError_t launch_kv_store(const IO* src, __half* cache, int n_vals, const int* positions, int pos0, long long T,
                            int kv_stride, int kv_shift, long long kv_bstride, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (!src || !cache || n_vals <= 0 || T <= 0 || kv_shift < 0 || kv_shift > 30 || kv_stride < n_vals || kv_bstride < 0 ||
        (!positions && pos0 < 0))
        return cudaErrorInvalidValue;
    const bool vec = n_vals % 8 == 0 && al16(src) && al16(cache) && kv_stride % 8 == 0 && kv_bstride % 8 == 0;
    const long long work = T * (vec ? n_vals / 8 : n_vals), cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_kv_store_f16<IO, true><<<(unsigned)grid, 256, 0, stream>>>(src, cache, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride);
    else k_kv_store_f16<IO, false><<<(unsigned)grid, 256, 0, stream>>>(src, cache, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride);
    return launched();
}

template <typename IO>
cudaError_t launch_kv_store_q(const IO* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                              int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, int rot,
                              cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (!src || !cache || n_vals <= 0 || n_vals % 32 != 0 || T <= 0 || kv_shift < 0 || kv_shift > 30 || kv_stride <= 0 ||
        kv_bstride < 0 || (!positions && pos0 < 0) || (kv_quant != 1 && kv_quant != 2) ||
        (rot != 0 && ((rot != 64 && rot != 128 && rot != 256 && rot != 512) || n_vals % rot != 0)))
        return cudaErrorInvalidValue;
    // the row must hold n_vals values and their scales: d_row = kv_stride * 32 / 17 (or / 9), as src/attention.hip:50
    const long long d_row = (long long)kv_stride * 32 / (kv_quant == 2 ? 9 : 17);
    const long long need = kv_quant == 2 ? d_row / 2 + n_vals / 32 * 2 : d_row + n_vals / 32 * 2;
    if (n_vals > d_row || need > (long long)kv_stride * 2 || (kv_quant == 2 ? d_row / 2 : d_row) % 2 != 0)
        return cudaErrorInvalidValue;
    // a thread writes its 8 values as one 8-byte (Q8_0) or 4-byte (Q4_0) word: rows must start on such a boundary
    // (the reference's rows, d_row % 256 == 0, are multiples of 272 and 144 bytes)
    const int unit = kv_quant == 1 ? 4 : 2;   // in fp16 units
    if (!al16(src) || kv_stride % unit != 0 || kv_bstride % unit != 0 ||
        (reinterpret_cast<uintptr_t>(cache) & (size_t)(2 * unit - 1)) != 0)
        return cudaErrorInvalidValue;
    constexpr int U = 2;
    const long long octets = T * (n_vals / 8), cap = resident_ctas(256) * 8;
    long long grid = (octets + 256 * U - 1) / (256 * U);
    if (grid > cap) grid = cap;
    __half* c = reinterpret_cast<__half*>(cache);
    {   // Rotated rows and 16-bit sources take the block-per-lane kernel (measured on 262,144 x 1,024 values, fraction of
        // the copy bandwidth, 8-per-lane -> block-per-lane: bf16 Q8_0 0.68 -> 1.03, bf16 Q4_0 0.47 -> 0.91, rotated fp32
        // 0.52 -> 0.75 and 0.43 -> 0.67); fp32 sources without rotation stay on the 8-per-lane one (0.96 / 0.90 against
        // 0.79 / 0.75: a lane's 128-byte run costs the fp32 loads their sector efficiency)
        const bool ok32 = kv_stride % 8 == 0 && kv_bstride % 8 == 0 && al16(cache);
        if (ok32 && (rot || sizeof(IO) == 2)) {
            const long long nblk = T * (n_vals / 32), cap32 = resident_ctas(128) * 8;
            long long g32 = (nblk + 127) / 128;
            if (g32 > cap32) g32 = cap32;
            // (rotated fp32 rows fetch the warp's span as consecutive chunks: 0.58 -> 0.75 and 0.54 -> 0.67; for 16-bit
            // sources the lanes' own 64-byte runs are faster, 1.03 / 0.91 against 0.94 / 0.82)
#define KVQ32(KQ, R) k_kv_store_q32<IO, KQ, R, (R && sizeof(IO) == 4)><<<(unsigned)g32, 128, 0, stream>>>(src, c, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride, rot)
            if (kv_quant == 1) { if (rot) KVQ32(1, true); else KVQ32(1, false); }
            else { if (rot) KVQ32(2, true); else KVQ32(2, false); }
#undef KVQ32
            return launched();
        }
    }
#define KVQ(KQ, R) k_kv_store_q<IO, KQ, U, R><<<(unsigned)grid, 256, 0, stream>>>(src, c, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride, rot)
    if (kv_quant == 1) { if (rot) KVQ(1, true); else KVQ(1, false); }
    else { if (rot) KVQ(2, true); else KVQ(2, false); }
#undef KVQ
    return launched();
}

template <typename IO>
cudaError_t launch_hadamard(const IO* x, IO* out, long long rows, int D, int N, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (!x || !out || rows <= 0 || D <= 0 || (N != 64 && N != 128 && N != 256 && N != 512) || D % N != 0 || !al16(x) || !al16(out))
        return cudaErrorInvalidValue;
    // a lane per 32 values, the warp's span read and written as consecutive chunks (measured against 8 values per lane
    // with one more shuffle stage: blocks of 128 0.82 -> 0.97 of the copy bandwidth, blocks of 512 0.70 -> 0.85)
    const long long total = rows * D, cap = resident_ctas(128) * 8;
    long long grid = (total / 32 + 127) / 128;
    if (grid > cap) grid = cap;
    k_hadamard_rot32<IO><<<(unsigned)grid, 128, 0, stream>>>(x, out, total, N);
    return launched();
}

// ---------------------------------------------------------------- MoE grouping

// Up to this many entries one CTA groups the batch in shared memory (no scratch, one launch); beyond it the segment
// kernels take over
constexpr int MOE_SINGLE_CTA_MAX = 8192;
constexpr int MOE_MAX_SEGS = 1024;
constexpr int MOE_SCRATCH_SLOTS = 4;

// Scratch of the reference-named launcher, which has no scratch argument: a few slots used in turn, so that calls
// still queued on other streams do not meet each other's counters (a caller with more than MOE_SCRATCH_SLOTS long
// groupings in flight on one device passes its own scratch: gpu_moe_group_scratch)
__device__ int g_moe_scratch[MOE_SCRATCH_SLOTS][MOE_MAX_SEGS * MOE_MAX_EXPERTS];
std::atomic<unsigned> g_moe_slot{0};

// Segments of a batch of n entries: at most MOE_MAX_SEGS, each a multiple of 32 entries and at least 1024
int moe_segments(int n, int* seg_len) {
    long long len = ((long long)n + MOE_MAX_SEGS - 1) / MOE_MAX_SEGS;
    len = (len + 31) / 32 * 32;
    if (len < 1024) len = 1024;
    if (seg_len) *seg_len = (int)len;
    return (int)((n + len - 1) / len);
}

cudaError_t launch_moe_group(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows,
                             int* n_tiles, int* tile_e, int* tile_start, int* tile_n, int* scratch, size_t scratch_ints,
                             cudaStream_t stream) {
    const int n = T * n_used;
    if (n <= MOE_SINGLE_CTA_MAX) {
        k_moe_group<<<1, 1024, 0, stream>>>(ids, T, n_used, n_expert, tile, tok_rows, pair_rows, n_tiles, tile_e,
                                            tile_start, tile_n);
        return launched();
    }
    int seg_len = 0;
    const int n_segs = moe_segments(n, &seg_len);
    if (!scratch) {
        void* base = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&base, g_moe_scratch);
        if (e != cudaSuccess) return e;
        const unsigned slot = g_moe_slot.fetch_add(1, std::memory_order_relaxed) % MOE_SCRATCH_SLOTS;
        scratch = static_cast<int*>(base) + (size_t)slot * MOE_MAX_SEGS * MOE_MAX_EXPERTS;
    }
    (void)scratch_ints;
    const int ctas = (n_segs + MOE_SEG_WARPS - 1) / MOE_SEG_WARPS;
    k_moe_seg_count<<<ctas, 32 * MOE_SEG_WARPS, 0, stream>>>(ids, n, n_expert, seg_len, n_segs, scratch);
    cudaError_t e = launched();
    if (e != cudaSuccess) return e;
    k_moe_seg_scan<<<1, 1024, 0, stream>>>(n_expert, next_pow2(n_expert), tile, n_segs, scratch, n_tiles, tile_e, tile_start,
                                           tile_n);
    e = launched();
    if (e != cudaSuccess) return e;
    k_moe_seg_scatter<<<ctas, 32 * MOE_SEG_WARPS, 0, stream>>>(ids, n, n_used, n_expert, seg_len, n_segs, scratch, tok_rows,
                                                               pair_rows);
    return launched();
}

template <bool SIGMOID>
cudaError_t launch_router(const float* logits, const float* x, const float* w_shexp, const float* bias, int* ids,
                          float* wts, float* sg, int n_expert, int n_used, int n, long long T, int ids_stride, int norm,
                          float scale, cudaStream_t stream) {
    long long grid = (T + MOE_ROUTER_WARPS - 1) / MOE_ROUTER_WARPS;
    const long long cap = resident_ctas(32 * MOE_ROUTER_WARPS) * 4;
    if (grid > cap) grid = cap;
#define ROUTER(PL) k_moe_router<PL, SIGMOID><<<(unsigned)grid, 32 * MOE_ROUTER_WARPS, 0, stream>>>( \
        logits, x, w_shexp, bias, ids, wts, sg, n_expert, n_used, n, T, ids_stride, norm, scale)
    if (n_expert <= 32) ROUTER(1);
    else if (n_expert <= 64) ROUTER(2);
    else if (n_expert <= 128) ROUTER(4);
    else if (n_expert <= 256) ROUTER(8);
    else if (n_expert <= 512) ROUTER(16);
    else ROUTER(32);
#undef ROUTER
    return launched();
}

// ---------------------------------------------------------------- Gemma-4 norm chains, GEGLU, soft cap

// Rows of n fp32 values, n % 256 == 0 and n <= 4096 (src/gpu_ops.cpp:189,198): exactly tpr * vpt vectors
bool plan_chain(int n, int* tpr, int* vpt) {
    if (n <= 0 || n % 256 != 0 || n > 256 * 16) return false;
    const int nvec = n / 4;
    *vpt = nvec % 128 == 0 ? 4 : 2;
    *tpr = nvec / *vpt;
    return true;
}

// add_normed and gemma_attn_post run one row per CTA, like the residual add + RMSNorm: CTAs that retire and are replaced
// in row order keep the rows in flight next to each other in memory (65,536 rows of 4096: 0.97 -> 1.06 and 0.93 -> 1.05 of
// the copy bandwidth against a grid of resident CTAs walking strided rows).
cudaError_t launch_add_normed(const float* base, const float* a, const float* w, const float* scale, float* out, int n,
                              long long T, float eps, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    int tpr, vpt;
    if (T <= 0 || !plan_chain(n, &tpr, &vpt) || a == out || !base || !a || !w || !out || !al16(base) || !al16(a) ||
        !al16(w) || !al16(out))
        return cudaErrorInvalidValue;
    if (vpt == 4) {
        const long long grid = T < INT_MAX ? T : INT_MAX;   // one row per CTA: CTAs retire in row order
        k_add_normed<4><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(base, a, w, scale, out, n, T, eps);
    } else {
        const long long grid = T < INT_MAX ? T : INT_MAX;   // one row per CTA: CTAs retire in row order
        k_add_normed<2><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(base, a, w, scale, out, n, T, eps);
    }
    return launched();
}

cudaError_t launch_attn_post(const float* x, const float* a, const float* w_a, float* x_out, const float* w1, float* y1,
                             const float* w2, float* y2, int n, long long T, float eps, cudaStream_t stream) {
    int tpr, vpt;
    if (!plan_chain(n, &tpr, &vpt) || !x || !a || !w_a || !x_out || !w1 || !y1 || (w2 && !y2) || !al16(x) || !al16(a) ||
        !al16(w_a) || !al16(x_out) || !al16(w1) || !al16(y1) || (w2 && (!al16(w2) || !al16(y2))))
        return cudaErrorInvalidValue;
    if (vpt == 4) {
        const long long grid = T < INT_MAX ? T : INT_MAX;   // one row per CTA: CTAs retire in row order
        k_gemma_attn_post<4><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(x, a, w_a, x_out, w1, y1, w2, y2, n, T, eps);
    } else {
        const long long grid = T < INT_MAX ? T : INT_MAX;   // one row per CTA: CTAs retire in row order
        k_gemma_attn_post<2><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(x, a, w_a, x_out, w1, y1, w2, y2, n, T, eps);
    }
    return launched();
}

}  // namespace

// ================================================================ C ABI

extern "C" {

int gpu_ops_init(const char* co_path) {
    (void)co_path;
    if (g_ready.load(std::memory_order_acquire)) return 0;
    // the kernels are loadable on the current device iff their attributes can be read
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, k_swiglu<float, false, 4>) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    (void)ones_vector();  // one-time set-up of the current device (other devices: at their first use)
    g_ready.store(true, std::memory_order_release);
    return 0;
}

void gpu_ops_free(void) { g_ready.store(false, std::memory_order_release); }

cudaError_t gpu_add_rmsnorm(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, int T,
                            float eps, const qmatvec_q8* q8, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || (q8 && (n % 256 != 0 || (long long)n * T > q8->max_k)) || (add && x_out == x_in))
        return cudaErrorInvalidValue;
    // the side outputs are written by the norm kernel itself where the row shape allows (one launch); for the other
    // shapes, what is left is one more pass over y
    bool xh_done = false, q8_done = false;
    Q8Side side = {};
    if (q8) side = side_of(q8);
    const cudaError_t e = launch_add_rmsnorm<float, float>(x_in, add, x_out, w, y, n, T, eps, stream, q8 ? &side : nullptr,
                                                           &xh_done, &q8_done);
    if (e != cudaSuccess || !q8) return e;
    qmatvec_q8 rest = *q8;
    if (xh_done) rest.xh = nullptr;
    if (q8_done) rest.qK = nullptr;
    return launch_q8_side(y, (long long)n * T, &rest, stream);
}

cudaError_t gpu_swiglu(const float* g, const float* u, float* out, int n, const qmatvec_q8* q8, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (q8 && (n % 32 != 0 || n > q8->max_k)) return cudaErrorInvalidValue;
    bool xh_done = false, q8_done = false;
    Q8Side side = {};
    if (q8) side = side_of(q8);
    const cudaError_t e = launch_swiglu<float, false>(g, u, out, n, stream, q8 ? &side : nullptr, &xh_done, &q8_done);
    if (e != cudaSuccess || !q8 || n <= 0) return e;
    qmatvec_q8 rest = *q8;
    if (xh_done) rest.xh = nullptr;
    if (q8_done) rest.qK = nullptr;
    return launch_q8_side(out, n, &rest, stream);
}

cudaError_t gpu_add_normed(const float* base, const float* a, const float* w, const float* scale, float* out, int n, int T,
                           float eps, cudaStream_t stream) {
    return launch_add_normed(base, a, w, scale, out, n, T, eps, stream);
}

cudaError_t gpu_gemma_attn_post(const float* x, const float* a, const float* w_a, float* x_out, const float* w1, float* y1,
                                const qmatvec_q8* q8, const float* w2, float* y2, int n, int T, float eps,
                                cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || (q8 && (long long)n * T > q8->max_k) || x_out == x || x_out == a) return cudaErrorInvalidValue;
    const cudaError_t e = launch_attn_post(x, a, w_a, x_out, w1, y1, w2, y2, n, T, eps, stream);
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(y1, (long long)n * T, q8, stream);
}

cudaError_t gpu_gemma_ffn_post(const float* x, const float* mlp, const float* down, const float* wts, const int* ids,
                               const float* exp_scale, int n_used, const float* w1, const float* w2, const float* w_post,
                               const float* scale, float* x_out, const float* w_next, float* y, const qmatvec_q8* q8, int n,
                               int T, float eps, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    int tpr, vpt;
    if (T <= 0 || n_used <= 0 || !plan_chain(n, &tpr, &vpt) || (q8 && (long long)n * T > q8->max_k) || x_out == x ||
        !x || !mlp || !down || !wts || (exp_scale && !ids) || !w1 || !w2 || !w_post || !x_out || !w_next || !y ||
        !al16(x) || !al16(mlp) || !al16(down) || !al16(w1) || !al16(w2) || !al16(w_post) || !al16(x_out) ||
        !al16(w_next) || !al16(y))
        return cudaErrorInvalidValue;
    // two vectors per thread whatever the width: with four the kernel needs 128 registers, which leaves an SM 16 warps
    // (measured 0.67 of the copy peak; 62 registers and 32 warps this way: 0.72)
    (void)vpt;
    tpr = n / 8;
    {
        long long grid = persistent_grid(k_gemma_ffn_post<2>, tpr, 0);   // (one row per CTA measured the same: 0.72)
        k_gemma_ffn_post<2><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(x, mlp, down, wts, ids, exp_scale, n_used, w1, w2, w_post, scale, x_out, w_next, y, n, T, eps);
    }
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(y, (long long)n * T, q8, stream);
}

cudaError_t gpu_hc_norm(const float* res_in, float* res_out, const float* cur, const float* inject, const float* w, float* y,
                        int n, int hc, int T, float eps, const qmatvec_q8* q8, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    int tpr, vpt;
    if (T <= 0 || hc <= 0 || !plan_chain(n, &tpr, &vpt) || (q8 && (long long)n * hc * T > q8->max_k) || !res_in || !w ||
        !y || (cur && (!res_out || !inject)) || !al16(res_in) || !al16(w) || !al16(y) ||
        (cur && (!al16(cur) || !al16(res_out))))
        return cudaErrorInvalidValue;
    const long long rows = (long long)T * hc;
    if (vpt == 4) {
        long long grid = persistent_grid(k_hc_norm<4>, tpr, 0);
        k_hc_norm<4><<<(unsigned)(grid < rows ? grid : rows), tpr, 0, stream>>>(res_in, res_out, cur, inject, w, y, n, hc, rows, eps);
    } else {
        long long grid = persistent_grid(k_hc_norm<2>, tpr, 0);
        k_hc_norm<2><<<(unsigned)(grid < rows ? grid : rows), tpr, 0, stream>>>(res_in, res_out, cur, inject, w, y, n, hc, rows, eps);
    }
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(y, rows * n, q8, stream);
}

cudaError_t gpu_hc_lowrank(const float* lo, float* out, int n, int np, int T, int hc, const qmatvec_q8* q8,
                           cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n <= 0 || hc <= 0 || np < n || !lo || !out || (q8 && (np % 32 != 0 || (long long)np * T > q8->max_k)))
        return cudaErrorInvalidValue;
    const long long total = (long long)np * T, cap = resident_ctas(256) * 8;
    long long grid = (total + 255) / 256;
    if (grid > cap) grid = cap;
    k_hc_lowrank<<<(unsigned)grid, 256, 0, stream>>>(lo, out, n, np, T, 1.0f / (float)hc);
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(out, total, q8, stream);
}

cudaError_t gpu_hc_mix(const float* xn, const float* gate, float* out, int n, int hc, int T, const qmatvec_q8* q8,
                       cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n <= 0 || hc <= 0 || !xn || !gate || !out || (q8 && (n % 256 != 0 || (long long)n * T > q8->max_k)))
        return cudaErrorInvalidValue;
    const bool vec = n % 4 == 0 && al16(xn) && al16(gate) && al16(out);
    const long long work = (long long)T * (vec ? n / 4 : n), cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_hc_mix<true><<<(unsigned)grid, 256, 0, stream>>>(xn, gate, out, n, hc, T);
    else k_hc_mix<false><<<(unsigned)grid, 256, 0, stream>>>(xn, gate, out, n, hc, T);
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(out, (long long)n * T, q8, stream);
}

cudaError_t gpu_ple_gate(const float* key, const float* value, const float* res, const float* wk, const float* wq,
                         const float* wc, float* gated, float* normed, int n, int hc, int T, float eps,
                         cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    int tpr, vpt;
    if (T <= 0 || hc <= 0 || !plan_chain(n, &tpr, &vpt) || !key || !value || !res || !wk || !wq || !wc || !gated ||
        !normed || !al16(key) || !al16(value) || !al16(res) || !al16(wk) || !al16(wq) || !al16(wc) || !al16(gated) ||
        !al16(normed))
        return cudaErrorInvalidValue;
    if (vpt == 4) {
        long long grid = persistent_grid(k_ple_gate<4>, tpr, 0);
        k_ple_gate<4><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(key, value, res, wk, wq, wc, gated, normed, n, hc, T, eps);
    } else {
        long long grid = persistent_grid(k_ple_gate<2>, tpr, 0);
        k_ple_gate<2><<<(unsigned)(grid < T ? grid : T), tpr, 0, stream>>>(key, value, res, wk, wq, wc, gated, normed, n, hc, T, eps);
    }
    return launched();
}

cudaError_t gpu_mtp_concat(const float* e, const float* h, float* out, int n, int hc, int T, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || hc <= 0 || n <= 0 || !e || !h || !out) return cudaErrorInvalidValue;
    const bool vec = n % 4 == 0 && al16(e) && al16(h) && al16(out);
    const long long rows = (long long)T * hc, work = rows * (vec ? n / 2 : 2 * n), cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_mtp_concat<true><<<(unsigned)grid, 256, 0, stream>>>(e, h, out, n, hc, rows);
    else k_mtp_concat<false><<<(unsigned)grid, 256, 0, stream>>>(e, h, out, n, hc, rows);
    return launched();
}

cudaError_t gpu_mamba_gnorm(const float* y, const float* zx, long long ld, const float* w, float* out, int d_inner,
                            int n_group, int T, float eps, const qmatvec_q8* q8, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n_group <= 0 || d_inner <= 0 || d_inner % n_group != 0) return cudaErrorInvalidValue;
    const int gs = d_inner / n_group;
    if (gs % 256 != 0 || gs > 1024 || (q8 && (long long)d_inner * T > q8->max_k) || !y || !zx || !w || !out || ld < d_inner ||
        ld % 4 != 0 || !al16(y) || !al16(zx) || !al16(w) || !al16(out))
        return cudaErrorInvalidValue;
    const long long rows = (long long)T * n_group;
    long long grid = persistent_grid(k_mamba_gnorm, gs / 8, 0);
    k_mamba_gnorm<<<(unsigned)(grid < rows ? grid : rows), gs / 8, 0, stream>>>(y, zx, ld, w, out, d_inner, n_group, T, eps);
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(out, (long long)d_inner * T, q8, stream);
}

cudaError_t gpu_mamba_conv(const float* zx, long long ld, int x_off, float* conv_state, const float* w, const float* bias,
                           float* out, int conv_dim, int d_conv, int T, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || d_conv < 2 || d_conv > MAMBA_MAXC || conv_dim <= 0 || !zx || !conv_state || !w || !bias || !out ||
        x_off < 0 || ld < (long long)x_off + conv_dim)
        return cudaErrorInvalidValue;
    const bool vec = conv_dim % 4 == 0 && ld % 4 == 0 && x_off % 4 == 0 && al16(zx) && al16(out);
    const long long work = (long long)T * (vec ? conv_dim / 4 : conv_dim), cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_mamba_conv<4><<<(unsigned)grid, 256, 0, stream>>>(zx, ld, x_off, conv_state, w, bias, out, conv_dim, d_conv, T);
    else k_mamba_conv<1><<<(unsigned)grid, 256, 0, stream>>>(zx, ld, x_off, conv_state, w, bias, out, conv_dim, d_conv, T);
    const cudaError_t e = launched();
    if (e != cudaSuccess) return e;
    k_mamba_conv_state<<<(unsigned)((conv_dim + 255) / 256), 256, 0, stream>>>(zx, ld, x_off, conv_state, conv_dim, d_conv, T);
    return launched();
}

cudaError_t gpu_mamba_scan(float* state, const float* xbc, const float* zx, long long ld, int dt_off, const float* dt_b,
                           const float* A, const float* D, float* y, int n_head, int d_inner, int n_group, int T,
                           cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n_head <= 0 || d_inner != n_head * MAMBA_P || n_group <= 0 || n_head % n_group != 0 || !state || !xbc ||
        !zx || !dt_b || !A || !D || !y || dt_off < 0 || !al16(state) || !al16(xbc))
        return cudaErrorInvalidValue;
    k_mamba_scan<<<(unsigned)n_head * 4, 64, 0, stream>>>(state, xbc, zx, ld, dt_off, dt_b, A, D, y, n_head, d_inner, n_group, T);
    return launched();
}

cudaError_t gpu_ple_conv(const float* normed, const float* gated, float* res, float* state, const void* w, int m, int T,
                         int K, int dil, const deltanet_mid_states* state_mid, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || K < 1 || dil < 1 || m <= 0 || !normed || !gated || !res || !w || (K > 1 && !state))
        return cudaErrorInvalidValue;
    MidStates mid = {{nullptr, nullptr, nullptr}};
    if (state_mid) memcpy(&mid, state_mid, sizeof(mid));
    const bool vec = m % 4 == 0 && al16(normed) && al16(gated) && al16(res) && (K == 1 || al16(state));
    const long long work = (long long)T * (vec ? m / 4 : m), cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    const __half* wh = static_cast<const __half*>(w);
    if (vec) k_ple_conv<4><<<(unsigned)grid, 256, 0, stream>>>(normed, gated, res, state, wh, m, T, K, dil);
    else k_ple_conv<1><<<(unsigned)grid, 256, 0, stream>>>(normed, gated, res, state, wh, m, T, K, dil);
    const cudaError_t e = launched();
    if (e != cudaSuccess || K == 1) return e;
    k_ple_conv_state<<<(unsigned)((m + 255) / 256), 256, 0, stream>>>(normed, state, m, T, K, dil, mid);
    return launched();
}

cudaError_t gpu_moe_router(const float* logits, const float* x, const float* w_shexp, int* ids, float* wts, float* sg,
                           int n_expert, int n_used, int n, int T, cudaStream_t stream, int ids_stride) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (n_expert <= 0 || n_expert > MOE_MAX_EXPERTS || n_used <= 0 || n_used > MOE_MAX_USED || n_used > n_expert || T <= 0)
        return cudaErrorInvalidValue;
    if (ids_stride == 0) ids_stride = n_used;
    if (ids_stride < n_used || !logits || !ids || !wts || (w_shexp && (!x || !sg || n <= 0))) return cudaErrorInvalidValue;
    return launch_router<false>(logits, x, w_shexp, nullptr, ids, wts, sg, n_expert, n_used, n, T, ids_stride, 1, 1.0f,
                                stream);
}

cudaError_t gpu_moe_router_sigmoid(const float* logits, const float* bias, int* ids, float* wts, int n_expert, int n_used,
                                   int norm, float scale, int T, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n_expert <= 0 || n_expert > MOE_MAX_EXPERTS || n_used <= 0 || n_used > MOE_MAX_USED ||
        n_used > n_expert || !logits || !bias || !ids || !wts)
        return cudaErrorInvalidValue;
    return launch_router<true>(logits, nullptr, nullptr, bias, ids, wts, nullptr, n_expert, n_used, 0, T, n_used, norm,
                               scale, stream);
}

cudaError_t gpu_relu2(const float* in, float* out, int rows, int h, int stride, const qmatvec_q8* q8, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    const long long n = (long long)rows * h;
    if (rows <= 0 || h <= 0 || stride < h || n > INT_MAX || !in || !out || (q8 && (n % 32 != 0 || n > q8->max_k)))
        return cudaErrorInvalidValue;
    const bool vec = h % 4 == 0 && stride % 4 == 0 && al16(in) && al16(out);
    const long long work = vec ? n / 4 : n, cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_relu2<true><<<(unsigned)grid, 256, 0, stream>>>(in, out, rows, h, stride);
    else k_relu2<false><<<(unsigned)grid, 256, 0, stream>>>(in, out, rows, h, stride);
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(out, n, q8, stream);
}

cudaError_t gpu_moe_combine_scaled(const float* down, const float* wts, const float* shared, const float* sg,
                                   const int* ids, const float* exp_scale, float* out, int n_used, int n, int T,
                                   cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if ((exp_scale && !ids) || T <= 0 || n <= 0 || n_used <= 0 || !down || !out) return cudaErrorInvalidValue;
    const bool vec = n % 4 == 0 && al16(down) && al16(out) && (!shared || al16(shared));
    const long long work = (long long)T * (vec ? n / 4 : n), cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_moe_combine<true><<<(unsigned)grid, 256, 0, stream>>>(down, wts, shared, sg, out, n_used, n, T, ids, exp_scale);
    else k_moe_combine<false><<<(unsigned)grid, 256, 0, stream>>>(down, wts, shared, sg, out, n_used, n, T, ids, exp_scale);
    return launched();
}

cudaError_t gpu_moe_combine(const float* down, const float* wts, const float* shared, const float* sg, float* out,
                            int n_used, int n, int T, cudaStream_t stream) {
    return gpu_moe_combine_scaled(down, wts, shared, sg, nullptr, nullptr, out, n_used, n, T, stream);
}

cudaError_t gpu_geglu(const float* gate, const float* up, float* out, int rows, int h, int gate_stride, int up_stride,
                      const qmatvec_q8* q8, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    const long long n = (long long)rows * h;
    if (rows <= 0 || h <= 0 || gate_stride < h || up_stride < h || n > INT_MAX || !gate || !up || !out ||
        (q8 && (n % 32 != 0 || n > q8->max_k)))
        return cudaErrorInvalidValue;
    const bool vec = h % 4 == 0 && gate_stride % 4 == 0 && up_stride % 4 == 0 && al16(gate) && al16(up) && al16(out);
    const long long work = vec ? n / 4 : n, cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_geglu<true><<<(unsigned)grid, 256, 0, stream>>>(gate, up, out, rows, h, gate_stride, up_stride);
    else k_geglu<false><<<(unsigned)grid, 256, 0, stream>>>(gate, up, out, rows, h, gate_stride, up_stride);
    const cudaError_t e = launched();
    if (e != cudaSuccess || !q8) return e;
    return launch_q8_side(out, n, q8, stream);
}

cudaError_t gpu_softcap(float* x, int n, float cap, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (n <= 0 || !(cap > 0.0f) || !x) return cudaErrorInvalidValue;
    const bool vec = al16(x);
    const long long work = vec ? (n + 3) / 4 : n, cap_ctas = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap_ctas) grid = cap_ctas;
    if (vec) k_softcap<true><<<(unsigned)grid, 256, 0, stream>>>(x, n, cap);
    else k_softcap<false><<<(unsigned)grid, 256, 0, stream>>>(x, n, cap);
    return launched();
}

cudaError_t gpu_moe_group(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows,
                          int* n_tiles, int* tile_e, int* tile_start, int* tile_n, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n_used <= 0 || n_expert <= 0 || n_expert > MOE_MAX_EXPERTS || tile <= 0 ||
        (long long)T * n_used > INT_MAX)
        return cudaErrorInvalidValue;
    return launch_moe_group(ids, T, n_used, n_expert, tile, tok_rows, pair_rows, n_tiles, tile_e, tile_start, tile_n,
                            nullptr, 0, stream);
}

size_t gpu_moe_group_scratch_ints(int T, int n_used, int n_expert) {
    const long long n = (long long)T * n_used;
    if (T <= 0 || n_used <= 0 || n_expert <= 0 || n > INT_MAX || n <= MOE_SINGLE_CTA_MAX) return 0;
    return (size_t)moe_segments((int)n, nullptr) * (size_t)n_expert;
}

cudaError_t gpu_moe_group_scratch(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows,
                                  int* n_tiles, int* tile_e, int* tile_start, int* tile_n, int* scratch,
                                  size_t scratch_ints, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (T <= 0 || n_used <= 0 || n_expert <= 0 || n_expert > MOE_MAX_EXPERTS || tile <= 0 ||
        (long long)T * n_used > INT_MAX || scratch_ints < gpu_moe_group_scratch_ints(T, n_used, n_expert) ||
        (!scratch && gpu_moe_group_scratch_ints(T, n_used, n_expert) > 0))
        return cudaErrorInvalidValue;
    return launch_moe_group(ids, T, n_used, n_expert, tile, tok_rows, pair_rows, n_tiles, tile_e, tile_start, tile_n,
                            scratch, scratch_ints, stream);
}

cudaError_t gpu_add_rmsnorm_f32(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n,
                                long long T, float eps, cudaStream_t stream) {
    return launch_add_rmsnorm<float, float>(x_in, add, x_out, w, y, n, T, eps, stream);
}

cudaError_t gpu_add_rmsnorm_bf16(const uint16_t* x_in, const uint16_t* add, uint16_t* x_out, const float* w,
                                 uint16_t* y, int n, long long T, float eps, cudaStream_t stream) {
    return launch_add_rmsnorm<__nv_bfloat16, float>(
        reinterpret_cast<const __nv_bfloat16*>(x_in), reinterpret_cast<const __nv_bfloat16*>(add),
        reinterpret_cast<__nv_bfloat16*>(x_out), w, reinterpret_cast<__nv_bfloat16*>(y), n, T, eps, stream);
}

cudaError_t gpu_swiglu_f32(const float* g, const float* u, float* out, long long n, cudaStream_t stream) {
    return launch_swiglu<float, false>(g, u, out, n, stream);
}

cudaError_t gpu_swiglu_bf16(const uint16_t* g, const uint16_t* u, uint16_t* out, long long n, cudaStream_t stream) {
    return launch_swiglu<__nv_bfloat16, true>(reinterpret_cast<const __nv_bfloat16*>(g),
                                              reinterpret_cast<const __nv_bfloat16*>(u),
                                              reinterpret_cast<__nv_bfloat16*>(out), n, stream);
}

cudaError_t gpu_swiglu_rows(const float* gate, const float* up, float* out, long long rows, int h,
                            long long gate_stride, long long up_stride, cudaStream_t stream) {
    return launch_swiglu_rows<float, false>(gate, up, out, rows, h, gate_stride, up_stride, stream);
}

cudaError_t gpu_swiglu_rows_bf16(const uint16_t* gate, const uint16_t* up, uint16_t* out, long long rows, int h,
                                 long long gate_stride, long long up_stride, cudaStream_t stream) {
    return launch_swiglu_rows<__nv_bfloat16, true>(reinterpret_cast<const __nv_bfloat16*>(gate),
                                                   reinterpret_cast<const __nv_bfloat16*>(up),
                                                   reinterpret_cast<__nv_bfloat16*>(out), rows, h, gate_stride,
                                                   up_stride, stream);
}

cudaError_t gpu_qk_norm_rope(const float* qfull, const float* k, const float* q_norm, const float* k_norm,
                             float* q_out, float* k_out, int n_q, int n_kv, int head_dim, int n_rot, int rot_pairs,
                             const int* positions, int pos0, long long T, float freq_base, float eps, int gated,
                             int qk_norm, const float* freq_factors, cudaStream_t stream) {
    return launch_qk<float>(qfull, k, q_norm, k_norm, q_out, k_out, n_q, n_kv, head_dim, n_rot, rot_pairs, positions,
                            pos0, T, freq_base, eps, gated, qk_norm, freq_factors, stream);
}

cudaError_t gpu_qk_norm_rope_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                  uint16_t* q_out, uint16_t* k_out, int n_q, int n_kv, int head_dim, int n_rot,
                                  int rot_pairs, const int* positions, int pos0, long long T, float freq_base,
                                  float eps, int gated, int qk_norm, const float* freq_factors, cudaStream_t stream) {
    return launch_qk<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(qfull),
                                    reinterpret_cast<const __nv_bfloat16*>(k), q_norm, k_norm,
                                    reinterpret_cast<__nv_bfloat16*>(q_out), reinterpret_cast<__nv_bfloat16*>(k_out),
                                    n_q, n_kv, head_dim, n_rot, rot_pairs, positions, pos0, T, freq_base, eps, gated,
                                    qk_norm, freq_factors, stream);
}

cudaError_t gpu_rope_table(const int* positions, int pos0, long long T, int n_rot, int rot_pairs, float freq_base,
                           const float* freq_factors, float* cos_tab, float* sin_tab, cudaStream_t stream) {
    return launch_rope_table(positions, pos0, T, n_rot, rot_pairs, freq_base, freq_factors, cos_tab, sin_tab, stream);
}

cudaError_t gpu_qk_norm_rope_tab(const float* qfull, const float* k, const float* q_norm, const float* k_norm,
                                 float* q_out, float* k_out, int n_q, int n_kv, int head_dim, int n_rot,
                                 const float* cos_tab, const float* sin_tab, long long T, float eps, int gated,
                                 int qk_norm, cudaStream_t stream) {
    const RopeTables tabs = {cos_tab, sin_tab};
    return launch_qk<float>(qfull, k, q_norm, k_norm, q_out, k_out, n_q, n_kv, head_dim, n_rot, 0, nullptr, 0, T, 1.0f, eps,
                            gated, qk_norm, nullptr, stream, KvTarget{nullptr, 0, 0, 0}, &tabs);
}

cudaError_t gpu_qk_norm_rope_tab_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                      uint16_t* q_out, uint16_t* k_out, int n_q, int n_kv, int head_dim, int n_rot,
                                      const float* cos_tab, const float* sin_tab, long long T, float eps, int gated,
                                      int qk_norm, cudaStream_t stream) {
    const RopeTables tabs = {cos_tab, sin_tab};
    return launch_qk<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(qfull),
                                    reinterpret_cast<const __nv_bfloat16*>(k), q_norm, k_norm,
                                    reinterpret_cast<__nv_bfloat16*>(q_out), reinterpret_cast<__nv_bfloat16*>(k_out),
                                    n_q, n_kv, head_dim, n_rot, 0, nullptr, 0, T, 1.0f, eps, gated, qk_norm, nullptr, stream,
                                    KvTarget{nullptr, 0, 0, 0}, &tabs);
}

cudaError_t gpu_qk_norm_rope_tab_kv(const float* qfull, const float* k, const float* q_norm, const float* k_norm,
                                    float* q_out, uint16_t* k_cache, int kv_stride, int kv_shift, long long kv_bstride,
                                    int n_q, int n_kv, int head_dim, int n_rot, const float* cos_tab, const float* sin_tab,
                                    const int* positions, int pos0, long long T, float eps, int gated, int qk_norm,
                                    cudaStream_t stream) {
    const RopeTables tabs = {cos_tab, sin_tab};
    return launch_qk<float, true>(qfull, k, q_norm, k_norm, q_out, nullptr, n_q, n_kv, head_dim, n_rot, 0, positions, pos0, T,
                                  1.0f, eps, gated, qk_norm, nullptr, stream,
                                  KvTarget{reinterpret_cast<__half*>(k_cache), kv_stride, kv_shift, kv_bstride}, &tabs);
}

cudaError_t gpu_qk_norm_rope_tab_kv_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                         uint16_t* q_out, uint16_t* k_cache, int kv_stride, int kv_shift,
                                         long long kv_bstride, int n_q, int n_kv, int head_dim, int n_rot,
                                         const float* cos_tab, const float* sin_tab, const int* positions, int pos0,
                                         long long T, float eps, int gated, int qk_norm, cudaStream_t stream) {
    const RopeTables tabs = {cos_tab, sin_tab};
    return launch_qk<__nv_bfloat16, true>(reinterpret_cast<const __nv_bfloat16*>(qfull),
                                          reinterpret_cast<const __nv_bfloat16*>(k), q_norm, k_norm,
                                          reinterpret_cast<__nv_bfloat16*>(q_out), nullptr, n_q, n_kv, head_dim, n_rot, 0,
                                          positions, pos0, T, 1.0f, eps, gated, qk_norm, nullptr, stream,
                                          KvTarget{reinterpret_cast<__half*>(k_cache), kv_stride, kv_shift, kv_bstride},
                                          &tabs);
}

cudaError_t gpu_qk_norm_rope_kv(const float* qfull, const float* k, const float* q_norm, const float* k_norm, float* q_out,
                                uint16_t* k_cache, int kv_stride, int kv_shift, long long kv_bstride, int n_q, int n_kv,
                                int head_dim, int n_rot, int rot_pairs, const int* positions, int pos0, long long T,
                                float freq_base, float eps, int gated, int qk_norm, const float* freq_factors,
                                cudaStream_t stream) {
    return launch_qk<float, true>(qfull, k, q_norm, k_norm, q_out, nullptr, n_q, n_kv, head_dim, n_rot, rot_pairs, positions,
                                  pos0, T, freq_base, eps, gated, qk_norm, freq_factors, stream,
                                  KvTarget{reinterpret_cast<__half*>(k_cache), kv_stride, kv_shift, kv_bstride});
}

cudaError_t gpu_qk_norm_rope_kv_bf16(const uint16_t* qfull, const uint16_t* k, const float* q_norm, const float* k_norm,
                                     uint16_t* q_out, uint16_t* k_cache, int kv_stride, int kv_shift, long long kv_bstride,
                                     int n_q, int n_kv, int head_dim, int n_rot, int rot_pairs, const int* positions,
                                     int pos0, long long T, float freq_base, float eps, int gated, int qk_norm,
                                     const float* freq_factors, cudaStream_t stream) {
    return launch_qk<__nv_bfloat16, true>(reinterpret_cast<const __nv_bfloat16*>(qfull),
                                          reinterpret_cast<const __nv_bfloat16*>(k), q_norm, k_norm,
                                          reinterpret_cast<__nv_bfloat16*>(q_out), nullptr, n_q, n_kv, head_dim, n_rot,
                                          rot_pairs, positions, pos0, T, freq_base, eps, gated, qk_norm, freq_factors, stream,
                                          KvTarget{reinterpret_cast<__half*>(k_cache), kv_stride, kv_shift, kv_bstride});
}

cudaError_t gpu_attn_prep_f16(const float* qfull, const float* k, const float* v, const float* q_norm, const float* k_norm,
                              float* q_out, uint16_t* K, uint16_t* V, int kv_stride, int kv_shift, long long kv_bstride,
                              int n_q, int n_kv, int head_dim, int n_rot, int rot_pairs, const int* positions, int pos0,
                              long long T, float freq_base, float eps, int gated, int qk_norm, const float* freq_factors,
                              cudaStream_t stream) {
    const cudaError_t e = gpu_qk_norm_rope_kv(qfull, k, q_norm, k_norm, q_out, K, kv_stride, kv_shift, kv_bstride, n_q, n_kv,
                                              head_dim, n_rot, rot_pairs, positions, pos0, T, freq_base, eps, gated, qk_norm,
                                              freq_factors, stream);
    if (e != cudaSuccess) return e;
    return launch_kv_store<float>(v, reinterpret_cast<__half*>(V), n_kv * head_dim, positions, pos0, T, kv_stride, kv_shift,
                                  kv_bstride, stream);
}

cudaError_t gpu_attn_prep_f16_bf16(const uint16_t* qfull, const uint16_t* k, const uint16_t* v, const float* q_norm,
                                   const float* k_norm, uint16_t* q_out, uint16_t* K, uint16_t* V, int kv_stride,
                                   int kv_shift, long long kv_bstride, int n_q, int n_kv, int head_dim, int n_rot,
                                   int rot_pairs, const int* positions, int pos0, long long T, float freq_base, float eps,
                                   int gated, int qk_norm, const float* freq_factors, cudaStream_t stream) {
    const cudaError_t e = gpu_qk_norm_rope_kv_bf16(qfull, k, q_norm, k_norm, q_out, K, kv_stride, kv_shift, kv_bstride, n_q,
                                                   n_kv, head_dim, n_rot, rot_pairs, positions, pos0, T, freq_base, eps, gated,
                                                   qk_norm, freq_factors, stream);
    if (e != cudaSuccess) return e;
    return launch_kv_store<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(v), reinterpret_cast<__half*>(V),
                                          n_kv * head_dim, positions, pos0, T, kv_stride, kv_shift, kv_bstride, stream);
}

cudaError_t gpu_kv_store_f16(const float* src, uint16_t* cache, int n_vals, const int* positions, int pos0, long long T,
                             int kv_stride, int kv_shift, long long kv_bstride, cudaStream_t stream) {
    return launch_kv_store<float>(src, reinterpret_cast<__half*>(cache), n_vals, positions, pos0, T, kv_stride, kv_shift,
                                  kv_bstride, stream);
}

cudaError_t gpu_kv_store_f16_bf16(const uint16_t* src, uint16_t* cache, int n_vals, const int* positions, int pos0,
                                  long long T, int kv_stride, int kv_shift, long long kv_bstride, cudaStream_t stream) {
    return launch_kv_store<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(src), reinterpret_cast<__half*>(cache),
                                          n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride, stream);
}

cudaError_t gpu_kv_store_q(const float* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                           int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, cudaStream_t stream) {
    return launch_kv_store_q<float>(src, cache, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride, kv_quant, 0, stream);
}

cudaError_t gpu_kv_store_q_rot(const float* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                               int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, int rot_block,
                               cudaStream_t stream) {
    return launch_kv_store_q<float>(src, cache, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride, kv_quant,
                                    rot_block, stream);
}

cudaError_t gpu_kv_store_q_rot_bf16(const uint16_t* src, void* cache, int n_vals, const int* positions, int pos0,
                                    long long T, int kv_stride, int kv_shift, long long kv_bstride, int kv_quant,
                                    int rot_block, cudaStream_t stream) {
    return launch_kv_store_q<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(src), cache, n_vals, positions, pos0, T,
                                            kv_stride, kv_shift, kv_bstride, kv_quant, rot_block, stream);
}

cudaError_t gpu_hadamard_rot(const float* x, float* out, long long rows, int D, int block, cudaStream_t stream) {
    return launch_hadamard<float>(x, out, rows, D, block, stream);
}

cudaError_t gpu_hadamard_rot_bf16(const uint16_t* x, uint16_t* out, long long rows, int D, int block, cudaStream_t stream) {
    return launch_hadamard<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out),
                                          rows, D, block, stream);
}

cudaError_t gpu_kv_store_q_bf16(const uint16_t* src, void* cache, int n_vals, const int* positions, int pos0, long long T,
                                int kv_stride, int kv_shift, long long kv_bstride, int kv_quant, cudaStream_t stream) {
    return launch_kv_store_q<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(src), cache, n_vals, positions, pos0, T,
                                            kv_stride, kv_shift, kv_bstride, kv_quant, 0, stream);
}

cudaError_t gpu_embed_rows(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens, float* out,
                           int E, long long T, float scale, int* bad_row, cudaStream_t stream) {
    return launch_embed<float>(type, table, row_bytes, vocab, tokens, out, E, T, scale, bad_row, stream);
}

cudaError_t gpu_embed_rows_bf16(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens,
                                uint16_t* out, int E, long long T, float scale, int* bad_row, cudaStream_t stream) {
    return launch_embed<__nv_bfloat16>(type, table, row_bytes, vocab, tokens, reinterpret_cast<__nv_bfloat16*>(out), E,
                                       T, scale, bad_row, stream);
}

cudaError_t gpu_embed_rows_host_ids(int type, const void* table, size_t row_bytes, int vocab,
                                    const int32_t* tokens_host, int32_t* tokens_dev, float* out, int E, long long T,
                                    float scale, int* bad_row, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (!tokens_host || !tokens_dev || T <= 0) return cudaErrorInvalidValue;
    for (long long t = 0; t < T; ++t)
        if (tokens_host[t] < 0 || tokens_host[t] >= vocab) return cudaErrorInvalidValue;
    const cudaError_t e =
        cudaMemcpyAsync(tokens_dev, tokens_host, (size_t)T * sizeof(int32_t), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
    return launch_embed<float>(type, table, row_bytes, vocab, tokens_dev, out, E, T, scale, bad_row, stream);
}

cudaError_t gpu_rmsnorm_f16(const uint16_t* x, const uint16_t* gamma, uint16_t* y, int n_tokens, int n_embd, float eps,
                            cudaStream_t stream) {
    return launch_add_rmsnorm<__half, __half>(reinterpret_cast<const __half*>(x), nullptr, nullptr,
                                              reinterpret_cast<const __half*>(gamma), reinterpret_cast<__half*>(y),
                                              n_embd, n_tokens, eps, stream);
}

cudaError_t gpu_rope_rotate_half_f16(const uint16_t* x, const float* ctab, const float* stab, uint16_t* y, int n_rows,
                                     int half_dim, cudaStream_t stream) {
    if (!g_ready.load(std::memory_order_acquire)) return cudaErrorInvalidDeviceFunction;
    if (n_rows <= 0 || half_dim <= 0 || !x || !y || !ctab || !stab) return cudaErrorInvalidValue;
    const __half* xh = reinterpret_cast<const __half*>(x);
    __half* yh = reinterpret_cast<__half*>(y);
    const bool vec = half_dim % 8 == 0 && al16(x) && al16(y) && al16(ctab) && al16(stab);
    const long long work = vec ? (long long)n_rows * (half_dim / 8) : (long long)n_rows * half_dim;
    const long long cap = resident_ctas(256) * 8;
    long long grid = (work + 255) / 256;
    if (grid > cap) grid = cap;
    if (vec) k_rope_rotate_half_f16_vec<<<(unsigned)grid, 256, 0, stream>>>(xh, ctab, stab, yh, n_rows, half_dim);
    else k_rope_rotate_half_f16<<<(unsigned)grid, 256, 0, stream>>>(xh, ctab, stab, yh, n_rows, half_dim);
    return launched();
}

unsigned long long b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* b200_build_arch(void) { return "sm_100a"; }

}  // extern "C"
