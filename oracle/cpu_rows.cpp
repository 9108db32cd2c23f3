// cpu_rows.cpp -- row-parallel CPU runner for the layer ops: TEST INFRASTRUCTURE ONLY (parity checker and the
// timed CPU baseline), never part of the product library.
//
// Built twice from this one file:
//   -DUSE_REF : the per-row work is done by the reference's own functions, compiled from the reference's source
//               tree where it lies (qwen_rmsnorm / qwen_rope_neox, src/qwen_ops.cpp:8-24; qwen_silu,
//               src/qwen_ops.h:47; qt_to_float, src/quant_types.cpp:641-646)  -> oracle/_ref/libref_cpu.so
//   otherwise : by the restatement in oracle_ops.c                             -> oracle/liboracle.so
// Both export the same cpu_* entry points, so a caller times or checks either with the same code. The loops
// around the per-row functions follow the reference's callers: the gather loop of src/qwen_model.cpp:980-986,
// the residual add of src/gpu_ops.hip:36,50-53, and qk_ref of tests/forward_verify.cpp:835-853.

#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

#ifdef USE_REF
#include "qwen_ops.h"
#include "quant_types.h"
static inline void row_rmsnorm(const float* x, const float* w, float* y, int n, float eps) { qwen_rmsnorm(x, w, y, n, eps); }
static inline void row_rope(float* v, int n_rot, int pos, float base) { qwen_rope_neox(v, n_rot, pos, base); }
static inline float one_silu(float x) { return qwen_silu(x); }
static inline int row_to_float(int type, const void* src, float* dst, int64_t n) { return qt_to_float(type, src, dst, n); }
extern "C" {
// the reference's C++-linkage functions under C names, for ctypes
void ref_qwen_rmsnorm(const float* x, const float* w, float* y, int n, float eps) { qwen_rmsnorm(x, w, y, n, eps); }
void ref_qwen_rope_neox(float* v, int n_rot, int pos, float base) { qwen_rope_neox(v, n_rot, pos, base); }
float ref_qwen_silu(float x) { return qwen_silu(x); }
int cpu_is_reference(void) { return 1; }
}
#else
#include "oracle_ops.h"
static inline void row_rmsnorm(const float* x, const float* w, float* y, int n, float eps) { orc_rmsnorm(x, w, y, n, eps); }
static inline void row_rope(float* v, int n_rot, int pos, float base) { orc_rope_neox(v, n_rot, pos, base); }
static inline float one_silu(float x) { return orc_silu(x); }
static inline int row_to_float(int type, const void* src, float* dst, int64_t n) { return orc_to_float(type, src, dst, n); }
extern "C" int cpu_is_reference(void) { return 0; }
#endif

// Runs fn(begin, end) over [0, total) cut into contiguous ranges, one per thread
template <class F>
static void parallel_rows(int64_t total, int nthreads, F fn) {
    if (nthreads <= 1 || total <= 1) { fn((int64_t)0, total); return; }
    nthreads = (int)std::min<int64_t>(nthreads, total);
    std::vector<std::thread> th;
    th.reserve(nthreads);
    for (int i = 0; i < nthreads; ++i) {
        const int64_t b = total * i / nthreads, e = total * (i + 1) / nthreads;
        th.emplace_back([=] { fn(b, e); });
    }
    for (auto& t : th) t.join();
}

extern "C" {

int cpu_hardware_threads(void) { return (int)std::thread::hardware_concurrency(); }

void cpu_add_rmsnorm(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, int T,
                     float eps, int nthreads) {
    parallel_rows(T, nthreads, [=](int64_t b, int64_t e) {
        for (int64_t t = b; t < e; ++t) {
            const float* xi = x_in + t * n;
            if (add) {
                float* xo = x_out + t * n;
                const float* a = add + t * n;
                for (int i = 0; i < n; ++i) xo[i] = xi[i] + a[i];
                xi = xo;
            }
            row_rmsnorm(xi, w, y + t * n, n, eps);
        }
    });
}

void cpu_swiglu(const float* g, const float* u, float* out, int64_t n, int nthreads) {
    parallel_rows(n, nthreads, [=](int64_t b, int64_t e) {
        for (int64_t i = b; i < e; ++i) out[i] = one_silu(g[i]) * u[i];
    });
}

// Full NeoX RoPE over n_rot dims at each row's position (positions NULL: pos0 + t), after the per-head RMSNorm
// when do_norm is set. Q heads are read at stride 2 D when gated.
void cpu_qk_norm_rope(const float* qfull, const float* k, const float* q_norm, const float* k_norm, float* q_out,
                      float* k_out, int n_q, int n_kv, int D, int n_rot, const int* positions, int pos0, int T,
                      float freq_base, float eps, int gated, int do_norm, int nthreads) {
    const int qs = gated ? 2 * D : D;
    parallel_rows(T, nthreads, [=](int64_t b, int64_t e) {
        for (int64_t t = b; t < e; ++t) {
            const int pos = positions ? positions[t] : pos0 + (int)t;
            for (int h = 0; h < n_q + n_kv; ++h) {
                const bool isq = h < n_q;
                const int hh = isq ? h : h - n_q;
                const float* src = isq ? qfull + (t * n_q + hh) * qs : k + (t * n_kv + hh) * D;
                float* dst = isq ? q_out + (t * n_q + hh) * D : k_out + (t * n_kv + hh) * D;
                if (do_norm) row_rmsnorm(src, isq ? q_norm : k_norm, dst, D, eps);
                else if (dst != src) memcpy(dst, src, (size_t)D * sizeof(float));
                if (n_rot > 0) row_rope(dst, n_rot, pos, freq_base);
            }
        }
    });
}

// Returns 0, or -1 if any token id is out of range or the type cannot be decoded (nothing is promised about out then)
int cpu_embed_rows(int type, const void* table, size_t row_bytes, int vocab, const int32_t* tokens, float* out, int E,
                   int T, float scale, int nthreads) {
    std::atomic<int> bad(0);
    parallel_rows(T, nthreads, [=, &bad](int64_t b, int64_t e) {
        for (int64_t t = b; t < e; ++t) {
            if (tokens[t] < 0 || tokens[t] >= vocab) { bad = 1; return; }
            float* o = out + t * E;
            if (row_to_float(type, (const char*)table + (size_t)tokens[t] * row_bytes, o, E) != 0) { bad = 1; return; }
            if (scale != 1.0f)
                for (int i = 0; i < E; ++i) o[i] *= scale;
        }
    });
    return bad ? -1 : 0;
}

}  // extern "C"
