// moe_router.cuh -- the MoE routers that produce what gpu_moe_group and gpu_moe_combine consume, after the reference's
// moe_router (src/gpu_ops.hip:118-241, softmax gating as llama.cpp's build_moe_ffn) and moe_router_sigmoid (:692-824):
//   softmax: p = softmax(logits[t]); the n_used largest p in descending order (ties to the lower expert index);
//            weights p / max(sum of the selected p, 6.103515625e-5); optionally the shared expert's gate
//            sg[t] = sigmoid(x[t] . w_shexp), and ids[t][n_used] = -1 when the ids rows are wider than n_used
//   sigmoid: p = sigmoid(logits[t]); the n_used largest p + bias; weights p (without the bias), divided by
//            max(sum, 6.103515625e-5) if norm, times scale
// One WARP per token (the reference spends a 256-thread CTA): lane l holds experts l + 32 j in registers, the
// softmax reductions and the n_used argmax rounds are shuffles, and a CTA's 8 warps work on 8 tokens at once. The only
// row-sized traffic is the gate's dot product, x [T][n]: 16-byte loads, four per lane in flight, four fp32 chains per
// lane combined in double (a fixed order, so the result does not depend on the launch shape).

#ifndef B200_MOE_ROUTER_CUH
#define B200_MOE_ROUTER_CUH

#include "common.cuh"

namespace b200 {

#define MOE_ROUTER_WARPS 8
#define MOE_MAX_USED 64

// The selection shared by both routers. v: this lane's keys (experts lane + 32 j; -inf where there is none). Round r
// takes the largest remaining key (lowest expert index among equals) and leaves its expert and its weight in lane
// r & 31 (rounds 0..31 in id0 / w0, rounds 32..63 in id1 / w1). The weight is the key itself (softmax) or
// sigmoid(lg[expert]), evaluated again by the same instructions that made the key, so the same bits (SIGMOID).
template <int PL, bool SIGMOID>
__device__ __forceinline__ void router_rounds(float (&v)[PL], const float* lg, int n_used, int lane, int& id0, float& w0,
                                              int& id1, float& w1) {
    for (int r = 0; r < n_used; ++r) {
        float bv = v[0];
        int bj = 0;
#pragma unroll
        for (int j = 1; j < PL; ++j)
            if (v[j] > bv) { bv = v[j]; bj = j; }   // strict: the lowest index among equals
        int be = lane + 32 * bj;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oe = __shfl_xor_sync(0xffffffffu, be, off);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        const float bw = SIGMOID ? __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lg[be]))) : bv;
        if (lane == (r & 31)) {
            if (r < 32) { id0 = be; w0 = bw; }
            else { id1 = be; w1 = bw; }
        }
        if ((be & 31) == lane) {
#pragma unroll
            for (int j = 0; j < PL; ++j)
                if (j == (be >> 5)) v[j] = -INFINITY;
        }
    }
}

// Weights of the selected experts: w_r / max(sum, 2^-14) (the sum in selection order, fp32) when norm, times scale
// when scale != 1; ids and weights written by the lanes that hold them
__device__ __forceinline__ void router_write(int id0, float w0, int id1, float w1, int n_used, int lane, int norm,
                                             float scale, int* ids_row, float* wts_row) {
    float ws = 0.0f;
    for (int r = 0; r < n_used; ++r) {
        const float a = __shfl_sync(0xffffffffu, w0, r & 31), b = __shfl_sync(0xffffffffu, w1, r & 31);
        ws = __fadd_rn(ws, r < 32 ? a : b);
    }
    ws = fmaxf(ws, 6.103515625e-5f);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = lane + 32 * h;
        if (r < n_used) {
            float w = h ? w1 : w0;
            if (norm) w = __fdiv_rn(w, ws);
            if (scale != 1.0f) w = __fmul_rn(w, scale);
            ids_row[r] = h ? id1 : id0;
            wts_row[r] = w;
        }
    }
}

// x[t] . w over n values by one warp
__device__ __forceinline__ float warp_dot(const float* x, const float* w, int n, int lane) {
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    if ((n & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0) {
        const int nv = n >> 2;
        for (int i0 = 0; i0 < nv; i0 += 128) {      // four vectors per lane per step
            uint4 rx[4], rw[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * 32 + lane;
                if (i < nv) {
                    rx[k] = ld_stream(reinterpret_cast<const uint4*>(x) + i);
                    rw[k] = __ldg(reinterpret_cast<const uint4*>(w) + i);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (i0 + k * 32 + lane < nv) {
                    a0 = fmaf(__uint_as_float(rx[k].x), __uint_as_float(rw[k].x), a0);
                    a1 = fmaf(__uint_as_float(rx[k].y), __uint_as_float(rw[k].y), a1);
                    a2 = fmaf(__uint_as_float(rx[k].z), __uint_as_float(rw[k].z), a2);
                    a3 = fmaf(__uint_as_float(rx[k].w), __uint_as_float(rw[k].w), a3);
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) a0 = fmaf(x[i], w[i], a0);
    }
    return (float)group_sum(((double)a0 + (double)a1) + ((double)a2 + (double)a3), 32);
}

template <int PL, bool SIGMOID>
__global__ void __launch_bounds__(32 * MOE_ROUTER_WARPS)
k_moe_router(const float* logits, const float* x, const float* w_shexp, const float* bias, int* ids, float* wts, float* sg,
             int n_expert, int n_used, int n, long long T, int ids_stride, int norm, float scale) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * MOE_ROUTER_WARPS;
    for (long long t = (long long)blockIdx.x * MOE_ROUTER_WARPS + (threadIdx.x >> 5); t < T; t += warps) {
        const float* lg = logits + t * n_expert;
        float v[PL];
        if (SIGMOID) {
#pragma unroll
            for (int j = 0; j < PL; ++j) {
                const int e = lane + 32 * j;
                v[j] = e < n_expert ? __fadd_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lg[e]))), bias[e]) : -INFINITY;
            }
        } else {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < PL; ++j) {
                const int e = lane + 32 * j;
                v[j] = e < n_expert ? lg[e] : -INFINITY;
                mx = fmaxf(mx, v[j]);
            }
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            double sum = 0.0;
#pragma unroll
            for (int j = 0; j < PL; ++j) {
                v[j] = lane + 32 * j < n_expert ? expf(__fsub_rn(v[j], mx)) : 0.0f;
                sum += (double)v[j];
            }
            const float inv = __fdiv_rn(1.0f, (float)group_sum(sum, 32));
#pragma unroll
            for (int j = 0; j < PL; ++j) v[j] = lane + 32 * j < n_expert ? __fmul_rn(v[j], inv) : -INFINITY;
        }
        int id0 = 0, id1 = 0;
        float w0 = 0.0f, w1 = 0.0f;
        router_rounds<PL, SIGMOID>(v, lg, n_used, lane, id0, w0, id1, w1);
        router_write(id0, w0, id1, w1, n_used, lane, SIGMOID ? norm : 1, SIGMOID ? scale : 1.0f, ids + t * ids_stride,
                     wts + t * n_used);
        if (!SIGMOID) {
            if (lane == 0 && ids_stride > n_used) ids[t * ids_stride + n_used] = -1;   // the shared expert's slot
            if (w_shexp) {   // uniform
                const float d = warp_dot(x + t * n, w_shexp, n, lane);
                if (lane == 0) sg[t] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-d)));
            }
        }
    }
}

// out [rows][h] = max(x, 0)^2, row r of x at in + r * stride (src/gpu_ops.hip:826-838). VEC: h, stride and the bases
// multiples of four values
template <bool VEC>
__global__ void __launch_bounds__(256)
k_relu2(const float* in, float* out, long long rows, int h, long long stride) {
    const int per_row = VEC ? h / 4 : h;
    const long long total = rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / per_row;
        const int c = (int)(i - r * per_row);
        if (VEC) {
            float v[4];
            Io<float>::unpack(ld_stream(in + r * stride + c * 4), v);
#pragma unroll
            for (int e = 0; e < 4; ++e) { v[e] = fmaxf(v[e], 0.0f); v[e] = __fmul_rn(v[e], v[e]); }
            st_stream(out + r * (long long)h + c * 4, Io<float>::pack(v));
        } else {
            const float v = fmaxf(in[r * stride + c], 0.0f);
            out[i] = __fmul_rn(v, v);
        }
    }
}

}  // namespace b200

#endif  // B200_MOE_ROUTER_CUH
