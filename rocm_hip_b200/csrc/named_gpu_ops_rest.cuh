// named_gpu_ops_rest.cuh -- the other twenty kernels the reference's launchers ask the gpu_ops module for by name
// (src/gpu_ops.cpp:26-48), in the launch shapes and with the argument lists those launchers use (src/gpu_ops.cpp:88-300;
// kernels src/gpu_ops.hip:118-838), so that the reference's own gpu_ops.cpp, compiled unchanged against the hip/
// shims, runs on this module image. Included by named_kernels.cu. Compatibility kernels, one value per thread of a
// 256-thread group as the reference lays them out; the arithmetic is this library's (double sums of squares and dot
// products, 1/rms as the CPU reference forms it, every fp32 product and sum rounded on its own, accurate expf), i.e.
// the native launchers' results up to the summation order of the reductions.

#ifndef B200_NAMED_GPU_OPS_REST_CUH
#define B200_NAMED_GPU_OPS_REST_CUH

#include "moe_group.cuh"
#include "moe_router.cuh"
#include "stream_ops.cuh"
#include "window_ops.cuh"

namespace {

#define NAMED_MAXV 16   // 256-value slices of a row held per thread: rows of up to 4096 values

// Sum over the 256 threads; ends with a barrier so that the buffer can be used again at once
__device__ __forceinline__ double sum256(double v, double* part) {
    v = group_sum(v, 32);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += part[k];
    __syncthreads();
    return tot;
}

// 1/rms of the thread's slice values x[0 .. nb) of a row of n values
__device__ __forceinline__ float row_inv(const float (&x)[NAMED_MAXV], int nb, int n, float eps, double* part) {
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) ss = fma((double)x[j], (double)x[j], ss);
    return inv_rms(sum256(ss, part), 1.0 / (double)n, eps);
}

}  // namespace

extern "C" __global__ void __launch_bounds__(256)
moe_router(const float* logits, const float* x, const float* w_shexp, int* ids, float* wts, float* sg, int n_expert,
           int n_used, int n, int ids_stride) {
    // one token per block: warp 0 routes it exactly as the native kernel's warps do, all eight warps share the gate's dot
    __shared__ double part[8];
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    if (w_shexp) {   // uniform
        double d = 0.0;
        for (int i = threadIdx.x; i < n; i += 256) d += (double)__fmul_rn(x[(size_t)t * n + i], w_shexp[i]);
        const float dot = (float)sum256(d, part);
        if (threadIdx.x == 0) sg[t] = sigmoid_f(dot);
    }
    if (threadIdx.x >= 32) return;
    const float* lg = logits + (size_t)t * n_expert;
    float v[32];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < n_expert ? lg[e] : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    double sum = 0.0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        v[j] = lane + 32 * j < n_expert ? expf(__fsub_rn(v[j], mx)) : 0.0f;
        sum += (double)v[j];
    }
    const float inv = __fdiv_rn(1.0f, (float)group_sum(sum, 32));
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = lane + 32 * j < n_expert ? __fmul_rn(v[j], inv) : -INFINITY;
    int id0 = 0, id1 = 0;
    float w0 = 0.0f, w1 = 0.0f;
    router_rounds<32, false>(v, lg, n_used, lane, id0, w0, id1, w1);
    router_write(id0, w0, id1, w1, n_used, lane, 1, 1.0f, ids + (size_t)t * ids_stride, wts + (size_t)t * n_used);
    if (lane == 0 && ids_stride > n_used) ids[(size_t)t * ids_stride + n_used] = -1;
}

extern "C" __global__ void __launch_bounds__(256)
moe_router_sigmoid(const float* logits, const float* bias, int* ids, float* wts, int n_expert, int n_used, int norm,
                   float scale) {
    if (threadIdx.x >= 32) return;
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* lg = logits + (size_t)t * n_expert;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < n_expert ? __fadd_rn(sigmoid_f(lg[e]), bias[e]) : -INFINITY;
    }
    int id0 = 0, id1 = 0;
    float w0 = 0.0f, w1 = 0.0f;
    router_rounds<32, true>(v, lg, n_used, lane, id0, w0, id1, w1);
    router_write(id0, w0, id1, w1, n_used, lane, norm, scale, ids + (size_t)t * n_used, wts + (size_t)t * n_used);
}

extern "C" __global__ void __launch_bounds__(256)
moe_combine(const float* down, const float* wts, const float* shared, const float* sg, float* out, int n_used, int n,
            const int* ids, const float* exp_scale) {
    const int t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const float* d = down + (size_t)t * n_used * n + i;
    const float* w = wts ? wts + (size_t)t * n_used : nullptr;
    const int* e = exp_scale ? ids + (size_t)t * n_used : nullptr;
    float acc = 0.0f;
    for (int j = 0; j < n_used; ++j) {
        float v = d[(size_t)j * n];
        if (w) v = e ? __fmul_rn(__fmul_rn(v, exp_scale[e[j]]), w[j]) : __fmul_rn(w[j], v);
        acc = j == 0 ? v : __fadd_rn(acc, v);
    }
    const size_t at = (size_t)t * n + i;
    if (shared) acc = __fadd_rn(acc, (sg && w) ? __fmul_rn(shared[at], sg[t]) : shared[at]);
    out[at] = acc;
}

extern "C" __global__ void __launch_bounds__(1024)
moe_group(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows, int* n_tiles,
          int* tile_e, int* tile_start, int* tile_n) {
    // the launcher gives this kernel one block whatever the batch (src/gpu_ops.cpp:119-121)
    __shared__ int cnt[MOE_MAX_EXPERTS], run_pos[MOE_MAX_EXPERTS];
    __shared__ int wsum[2][32];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, n = T * n_used;
    cnt[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += 1024) {
        const int e = ids[i];
        if (e >= 0 && e < n_expert) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    const int c = tid < n_expert ? cnt[tid] : 0, nt = (c + tile - 1) / tile;
    int a = c, b = nt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int ua = __shfl_up_sync(0xffffffffu, a, d), ub = __shfl_up_sync(0xffffffffu, b, d);
        if (lane >= d) { a += ua; b += ub; }
    }
    if (lane == 31) { wsum[0][w] = a; wsum[1][w] = b; }
    __syncthreads();
    if (w == 0) {
        int x = wsum[0][lane], y = wsum[1][lane];
        const int x0 = x, y0 = y;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int ux = __shfl_up_sync(0xffffffffu, x, d), uy = __shfl_up_sync(0xffffffffu, y, d);
            if (lane >= d) { x += ux; y += uy; }
        }
        wsum[0][lane] = x - x0;
        wsum[1][lane] = y - y0;
    }
    __syncthreads();
    const int eo = wsum[0][w] + a - c, to = wsum[1][w] + b - nt;
    run_pos[tid] = eo;
    if (tid < n_expert) {
        for (int k = 0; k < nt; ++k) {
            tile_e[to + k] = tid;
            tile_start[to + k] = eo + k * tile;
            tile_n[to + k] = min(tile, c - k * tile);
        }
        if (tid == n_expert - 1) *n_tiles = to + nt;
    }
    __syncthreads();
    // entries in index order, 32 at a time by warp 0: ascending pair index inside every expert's run
    if (w == 0)
        for (int base = 0; base < n; base += 32) {
            const int i = base + lane;
            const int e = i < n ? ids[i] : -1;
            const bool ok = e >= 0 && e < n_expert;
            const unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
            const int rank = __popc(peers & ((1u << lane) - 1u));
            int p = 0;
            if (ok) p = run_pos[e] + rank;
            __syncwarp();
            if (ok && rank == 0) run_pos[e] += __popc(peers);
            __syncwarp();
            if (ok) {
                tok_rows[p] = i / n_used;
                pair_rows[p] = i;
            }
        }
}

extern "C" __global__ void __launch_bounds__(256)
hc_norm(const float* res_in, float* res_out, const float* cur, const float* inject, const float* w, float* y, int n, int hc,
        float eps, Q8Side o) {
    __shared__ double part[8];
    __shared__ Q8Scratch sh;
    const int r = blockIdx.y, t = r / hc, c = r % hc, tid = threadIdx.x, nb = n / 256;
    const bool split = gridDim.x > 1;     // the row spread over n / 256 blocks, each writing its own slice
    const float* x = res_in + (size_t)r * n;
    float v[NAMED_MAXV];
    const float wt = cur ? __fmul_rn(2.0f, sigmoid_f(__fmul_rn(inject[t * hc + c], __fdiv_rn(1.0f, (float)hc)))) : 0.0f;
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {
            const int k = tid + 256 * j;
            v[j] = x[k];
            if (cur) v[j] = __fadd_rn(v[j], __fmul_rn(cur[(size_t)t * n + k], wt));
        }
    const float inv = row_inv(v, nb, n, eps, part);
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb && (!split || j == (int)blockIdx.x)) {   // uniform
            const int k = tid + 256 * j;
            if (cur) res_out[(size_t)r * n + k] = v[j];
            const float out = __fmul_rn(__fmul_rn(v[j], inv), w[c * n + k]);
            y[(size_t)r * n + k] = out;
            if (q8_wanted(o)) q8_block_value(out, true, (long long)r * nb + j, tid, sh, o);
        }
}

extern "C" __global__ void __launch_bounds__(256)
hc_lowrank(const float* lo, float* out, int n, int np, int T, float scale, Q8Side o) {
    __shared__ Q8Scratch sh;
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    const long long t = i / np;
    const int k = (int)(i - t * np);
    const bool active = i < (long long)np * T;
    float v = 0.0f;
    if (active) {
        if (k < n) v = silu_f(__fmul_rn(lo[t * n + k], scale));
        out[i] = v;
    }
    if (q8_wanted(o)) q8_block_value(v, active, blockIdx.x, threadIdx.x, sh, o);
}

extern "C" __global__ void __launch_bounds__(256)
hc_mix(const float* xn, const float* gate, float* out, int n, int hc, Q8Side o) {
    __shared__ Q8Scratch sh;
    const int t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    float v = 0.0f;
    if (i < n) {
        const size_t base = (size_t)t * hc * n + i;
        for (int c = 0; c < hc; ++c) {
            const float p = __fmul_rn(xn[base + (size_t)c * n], sigmoid_f(gate[base + (size_t)c * n]));
            v = c == 0 ? p : __fadd_rn(v, p);
        }
        v = __fmul_rn(v, __fdiv_rn(1.0f, (float)hc));
        out[(size_t)t * n + i] = v;
    }
    if (q8_wanted(o)) q8_block_value(v, i < n, (long long)t * (n / 256) + blockIdx.x, threadIdx.x, sh, o);
}

extern "C" __global__ void __launch_bounds__(256)
mtp_concat(const float* e, const float* h, float* out, int n, int hc) {
    const int r = blockIdx.y, t = r / hc, i = blockIdx.x * 256 + threadIdx.x;
    if (i < 2 * n) out[(size_t)r * 2 * n + i] = i < n ? e[(size_t)t * n + i] : h[(size_t)r * n + i - n];
}

extern "C" __global__ void __launch_bounds__(256)
ple_gate(const float* key, const float* value, const float* res, const float* wk, const float* wq, const float* wc,
         float* gated, float* normed, int n, int hc, float eps) {
    __shared__ double part[8];
    const int t = blockIdx.x, tid = threadIdx.x, nb = n / 256;
    const float inv_sqrt_n = __fdiv_rn(1.0f, __fsqrt_rn((float)n));
    for (int c = 0; c < hc; ++c) {
        const size_t r = ((size_t)t * hc + c) * n;
        float kx[NAMED_MAXV], qx[NAMED_MAXV];
#pragma unroll
        for (int j = 0; j < NAMED_MAXV; ++j)
            if (j < nb) {
                kx[j] = key[r + tid + 256 * j];
                qx[j] = res[r + tid + 256 * j];
            }
        const float ik = row_inv(kx, nb, n, eps, part), iq = row_inv(qx, nb, n, eps, part);
        double d = 0.0;
#pragma unroll
        for (int j = 0; j < NAMED_MAXV; ++j)
            if (j < nb) {
                const int k = c * n + tid + 256 * j;
                d += (double)__fmul_rn(__fmul_rn(__fmul_rn(kx[j], ik), wk[k]), __fmul_rn(__fmul_rn(qx[j], iq), wq[k]));
            }
        const float s = __fmul_rn((float)sum256(d, part), inv_sqrt_n);
        const float mag = __fsqrt_rn(fmaxf(fabsf(s), 1e-6f));
        const float g = sigmoid_f(__fmul_rn(s > 0.0f ? 1.0f : (s < 0.0f ? -1.0f : 0.0f), mag));
#pragma unroll
        for (int j = 0; j < NAMED_MAXV; ++j)
            if (j < nb) kx[j] = __fmul_rn(value[(size_t)t * n + tid + 256 * j], g);
        const float ig = row_inv(kx, nb, n, eps, part);
#pragma unroll
        for (int j = 0; j < NAMED_MAXV; ++j)
            if (j < nb) {
                const int k = tid + 256 * j;
                gated[r + k] = kx[j];
                normed[r + k] = __fmul_rn(__fmul_rn(kx[j], ig), wc[c * n + k]);
            }
    }
}

extern "C" __global__ void __launch_bounds__(256)
ple_conv(const float* normed, const float* gated, float* res, float* state, const __half* w, int m, int T, int K, int dil,
         MidStates mid) {
    // one thread per channel walks the tokens (the launcher's shape, src/gpu_ops.cpp:175); the native launcher
    // spreads (token, channel) pairs over the device instead
    const int ch = blockIdx.x * 256 + threadIdx.x;
    if (ch >= m) return;
    const int H = (K - 1) * dil;
    for (int t = 0; t < T; ++t) {
        float acc = 0.0f;
        for (int k = 0; k < K; ++k) {
            const int j = t - (K - 1 - k) * dil;
            const float x = j >= 0 ? normed[(size_t)j * m + ch] : state[(size_t)(H + j) * m + ch];
            const float term = __fmul_rn(x, __half2float(w[(size_t)ch * K + k]));
            acc = k == 0 ? term : __fadd_rn(acc, term);
        }
        const size_t i = (size_t)t * m + ch;
        res[i] = __fadd_rn(res[i], __fadd_rn(gated[i], silu_f(acc)));
    }
    ple_conv_state_channel(normed, state, m, T, K, dil, mid, ch);
}

extern "C" __global__ void __launch_bounds__(256)
add_normed(const float* base, const float* a, const float* w, const float* scale, float* out, int n, float eps) {
    __shared__ double part[8];
    const size_t row = (size_t)blockIdx.x * n;
    const int t = threadIdx.x, nb = n / 256;
    float x[NAMED_MAXV];
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) x[j] = a[row + t + 256 * j];
    const float inv = row_inv(x, nb, n, eps, part), s = scale ? *scale : 1.0f;
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {
            const int k = t + 256 * j;
            out[row + k] = __fmul_rn(__fadd_rn(base[row + k], __fmul_rn(__fmul_rn(x[j], inv), w[k])), s);
        }
}

extern "C" __global__ void __launch_bounds__(256)
gemma_attn_post(const float* x, const float* a, const float* w_a, float* x_out, const float* w1, float* y1, Q8Side o1,
                const float* w2, float* y2, int n, float eps) {
    __shared__ double part[8];
    __shared__ Q8Scratch sh;
    const size_t row = (size_t)blockIdx.x * n;
    const int t = threadIdx.x, nb = n / 256;
    float v[NAMED_MAXV];
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) v[j] = a[row + t + 256 * j];
    const float ia = row_inv(v, nb, n, eps, part);
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {
            const int k = t + 256 * j;
            v[j] = __fadd_rn(x[row + k], __fmul_rn(__fmul_rn(v[j], ia), w_a[k]));
            x_out[row + k] = v[j];
        }
    const float inv = row_inv(v, nb, n, eps, part);
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {   // uniform
            const int k = t + 256 * j;
            const float vn = __fmul_rn(v[j], inv), y = __fmul_rn(vn, w1[k]);
            y1[row + k] = y;
            if (w2) y2[row + k] = __fmul_rn(vn, w2[k]);
            if (q8_wanted(o1)) q8_block_value(y, true, (long long)blockIdx.x * nb + j, t, sh, o1);
        }
}

extern "C" __global__ void __launch_bounds__(256)
gemma_ffn_post(const float* x, const float* mlp, const float* down, const float* wts, const int* ids, const float* exp_scale,
               int n_used, const float* w1, const float* w2, const float* w_post, const float* scale, float* x_out,
               const float* w_next, float* y, Q8Side o, int n, float eps) {
    __shared__ double part[8];
    __shared__ Q8Scratch sh;
    const int tk = blockIdx.x, t = threadIdx.x, nb = n / 256;
    const size_t row = (size_t)tk * n;
    float h[NAMED_MAXV], c[NAMED_MAXV];
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) h[j] = mlp[row + t + 256 * j];
    const float im = row_inv(h, nb, n, eps, part);
    const float* wt = wts + (size_t)tk * n_used;
    const int* e = ids + (size_t)tk * n_used;
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {
            const int k = t + 256 * j;
            h[j] = __fmul_rn(__fmul_rn(h[j], im), w1[k]);
            const float* d = down + (size_t)tk * n_used * n + k;
            float acc = 0.0f;
            for (int u = 0; u < n_used; ++u) {
                const float dv = d[(size_t)u * n];
                const float term = exp_scale ? __fmul_rn(__fmul_rn(dv, exp_scale[e[u]]), wt[u]) : __fmul_rn(wt[u], dv);
                acc = u == 0 ? term : __fadd_rn(acc, term);
            }
            c[j] = acc;
        }
    const float ic = row_inv(c, nb, n, eps, part);
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) h[j] = __fadd_rn(h[j], __fmul_rn(__fmul_rn(c[j], ic), w2[t + 256 * j]));
    const float ih = row_inv(h, nb, n, eps, part), sc = scale ? *scale : 1.0f;
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {
            const int k = t + 256 * j;
            h[j] = __fmul_rn(__fadd_rn(x[row + k], __fmul_rn(__fmul_rn(h[j], ih), w_post[k])), sc);
            x_out[row + k] = h[j];
        }
    const float inv = row_inv(h, nb, n, eps, part);
#pragma unroll
    for (int j = 0; j < NAMED_MAXV; ++j)
        if (j < nb) {   // uniform
            const int k = t + 256 * j;
            const float v = __fmul_rn(__fmul_rn(h[j], inv), w_next[k]);
            y[row + k] = v;
            if (q8_wanted(o)) q8_block_value(v, true, (long long)tk * nb + j, t, sh, o);
        }
}

extern "C" __global__ void __launch_bounds__(256)
mamba_conv(const float* zx, long long ld, int x_off, const float* conv_state, const float* w, const float* bias, float* out,
           int conv_dim, int d_conv) {
    const int c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y, ns = d_conv - 1;
    if (c >= conv_dim) return;
    float s = 0.0f;
    for (int i = 0; i <= ns; ++i) {
        const int tt = t - ns + i;
        const float h = tt >= 0 ? zx[(size_t)tt * ld + x_off + c] : conv_state[(size_t)c * ns + ns + tt];
        s = __fadd_rn(s, __fmul_rn(h, w[(size_t)c * d_conv + i]));
    }
    out[(size_t)t * conv_dim + c] = silu_f(__fadd_rn(s, bias[c]));
}

extern "C" __global__ void __launch_bounds__(256)
mamba_conv_state(const float* zx, long long ld, int x_off, float* conv_state, int conv_dim, int d_conv, int T) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < conv_dim) mamba_conv_state_channel(zx, ld, x_off, conv_state, c, d_conv, T);
}

extern "C" __global__ void __launch_bounds__(256)
mamba_scan(float* state, const float* xbc, const float* zx, long long ld, int dt_off, const float* dt_b, const float* A,
           const float* D, float* y, int d_inner, int n_group, int T) {
    // one head per block, 64 dims x 4 threads (src/gpu_ops.cpp:256); the native launcher cuts a head into four blocks
    mamba_scan_thread(state, xbc, zx, ld, dt_off, dt_b, A, D, y, (int)gridDim.x, d_inner, n_group, T, blockIdx.x,
                      threadIdx.x >> 2, threadIdx.x & 3);
}

extern "C" __global__ void __launch_bounds__(256)
mamba_gnorm(const float* y, const float* zx, long long ld, const float* w, float* out, int d_inner, float eps, Q8Side o) {
    __shared__ double part[8];
    __shared__ Q8Scratch sh;
    const int g = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, gs = d_inner / gridDim.x, nb = gs / 256;
    float v[NAMED_MAXV];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
        if (jj < nb) {
            const int k = g * gs + tid + 256 * jj;
            v[jj] = __fmul_rn(y[(size_t)t * d_inner + k], silu_f(zx[(size_t)t * ld + k]));
        }
    const float inv = row_inv(v, nb, gs, eps, part);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
        if (jj < nb) {   // uniform
            const int k = g * gs + tid + 256 * jj;
            const float r = __fmul_rn(__fmul_rn(v[jj], inv), w[k]);
            out[(size_t)t * d_inner + k] = r;
            if (q8_wanted(o)) q8_block_value(r, true, ((long long)t * d_inner + (long long)g * gs) / 256 + jj, tid, sh, o);
        }
}

extern "C" __global__ void __launch_bounds__(256)
relu2(const float* in, float* out, int n, int h, int stride, Q8Side o) {
    __shared__ Q8Scratch sh;
    const int i = blockIdx.x * 256 + threadIdx.x;
    float v = 0.0f;
    if (i < n) {
        const float r = fmaxf(in[(size_t)(i / h) * stride + i % h], 0.0f);
        v = __fmul_rn(r, r);
        out[i] = v;
    }
    if (q8_wanted(o)) q8_block_value(v, i < n, blockIdx.x, threadIdx.x, sh, o);
}

extern "C" __global__ void __launch_bounds__(256)
geglu(const float* gate, const float* up, float* out, int n, int h, int gs, int us, Q8Side o) {
    __shared__ Q8Scratch sh;
    const int i = blockIdx.x * 256 + threadIdx.x;
    float v = 0.0f;
    if (i < n) {
        const int r = i / h, c = i % h;
        v = gelu_tanh_mul(gate[(size_t)r * gs + c], up[(size_t)r * us + c]);
        out[i] = v;
    }
    if (q8_wanted(o)) q8_block_value(v, i < n, blockIdx.x, threadIdx.x, sh, o);
}

extern "C" __global__ void __launch_bounds__(256)
softcap(float* x, int n, float cap) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) x[i] = __fmul_rn(cap, tanhf(__fdiv_rn(x[i], cap)));
}

#endif  // B200_NAMED_GPU_OPS_REST_CUH
