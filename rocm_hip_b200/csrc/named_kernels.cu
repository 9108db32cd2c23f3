// named_kernels.cu -- the kernel entry points the reference looks up BY NAME in its code objects, for a caller that
// keeps the reference's own module-launch code (cuModuleLoadData + cuModuleGetFunction in place of
// hipModuleLoadData + hipModuleGetFunction). Same names, argument lists and launch geometry:
//   "add_rmsnorm"       grid (ceil(n / 256), T), block 256      src/gpu_ops.hip:24-56, launched at src/gpu_ops.cpp:76
//   "add_rmsnorm_rows"  grid T, block 256 (n % 256 == 0)        src/gpu_ops.hip:64-101, launched at src/gpu_ops.cpp:75
//   "swiglu"            grid ceil(n / 256), block 256           src/gpu_ops.hip:103-114, launched at src/gpu_ops.cpp:85
//   "rmsnorm"           grid n_tokens, block 32                 src/layernorm.hip:15-45, launched at tests/layernorm_verify.cpp:96
//   "rope_rotate_half"  grid n_rows, block 32                   src/rope_embedding.hip:18-37, tests/rope_verify.cpp:113
// The by-value struct of side-output pointers has the layout of the reference's Q8Out (src/q8_device.h:22-31).
// The reference's gpu_ops module holds twenty more names (moe_router ... softcap, src/gpu_ops.cpp:29-48) for model
// families outside this library's path; this image does not provide them.
// These are compatibility kernels in the reference's launch shapes (which re-read rows or use one warp per row); the
// library's own launchers (layer_ops.cu) use better-shaped kernels with the same arithmetic: double-precision sums
// of squares, 1/rms as the CPU reference forms it, products rounded separately. Built into gpu_ops.fatbin.

#include "common.cuh"
#include "q8_side.cuh"
#include "swiglu.cuh"

using namespace b200;

namespace {
__device__ __forceinline__ bool q8_wanted(const Q8Side& o) { return o.qK || o.xh; }
}

extern "C" __global__ void __launch_bounds__(256)
add_rmsnorm(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, float eps, Q8Side o) {
    __shared__ double part[32];
    __shared__ Q8Scratch sh;
    const size_t row = (size_t)blockIdx.y * n;
    x_in += row; x_out += row; y += row;
    if (add) add += row;
    const int t = threadIdx.x, i = blockIdx.x * 256 + t;
    double ss = 0.0;
    for (int k = t; k < n; k += 256) {   // every group sums the whole row, in the same order, so all get one scale
        const float v = add ? __fadd_rn(x_in[k], add[k]) : x_in[k];
        ss = fma((double)v, (double)v, ss);
    }
    const float inv = inv_rms(cta_sum(ss, part), 1.0 / (double)n, eps);
    const bool active = i < n;
    float v = 0.0f;
    if (active) {
        v = add ? __fadd_rn(x_in[i], add[i]) : x_in[i];
        if (add) x_out[i] = v;
        v = __fmul_rn(__fmul_rn(v, inv), w ? w[i] : 1.0f);
        y[i] = v;
    }
    if (q8_wanted(o)) q8_block_value(v, active, (long long)blockIdx.y * (n / 256) + blockIdx.x, t, sh, o);
}

extern "C" __global__ void __launch_bounds__(256)
add_rmsnorm_rows(const float* x_in, const float* add, float* x_out, const float* w, float* y, int n, float eps, Q8Side o) {
    __shared__ double part[32];
    __shared__ Q8Scratch sh;
    const size_t row = (size_t)blockIdx.x * n;
    x_in += row; x_out += row; y += row;
    if (add) add += row;
    const int t = threadIdx.x, nb = n / 256;
    double ss = 0.0;
    for (int j = 0; j < nb; ++j) {
        const int k = t + 256 * j;
        const float v = add ? __fadd_rn(x_in[k], add[k]) : x_in[k];
        if (add) x_out[k] = v;
        ss = fma((double)v, (double)v, ss);
    }
    const float inv = inv_rms(cta_sum(ss, part), 1.0 / (double)n, eps);
    for (int j = 0; j < nb; ++j) {   // (uniform trip count: q8_block_value synchronises the group)
        const int k = t + 256 * j;
        const float x = add ? x_out[k] : x_in[k];   // this thread wrote x_out[k] above
        const float v = __fmul_rn(__fmul_rn(x, inv), w ? w[k] : 1.0f);
        y[k] = v;
        if (q8_wanted(o)) q8_block_value(v, true, (long long)blockIdx.x * nb + j, t, sh, o);
    }
}

extern "C" __global__ void __launch_bounds__(256)
swiglu(const float* g, const float* u, float* out, int n, Q8Side o) {
    __shared__ Q8Scratch sh;
    const int i = blockIdx.x * 256 + threadIdx.x;
    float v = 0.0f;
    if (i < n) {
        v = silu_mul<false>(g[i], u[i]);
        out[i] = v;
    }
    if (q8_wanted(o)) q8_block_value(v, i < n, blockIdx.x, threadIdx.x, sh, o);
}

// FP16 rows, one block per token row; any blockDim that is a multiple of 32 up to 1024 (the reference launches 32)
extern "C" __global__ void rmsnorm(const __half* x, const __half* gamma, __half* y, int n_tokens, int n_embd, float eps) {
    __shared__ double part[32];
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const __half* xr = x + (size_t)t * n_embd;
    __half* yr = y + (size_t)t * n_embd;
    double ss = 0.0;
    for (int c = threadIdx.x; c < n_embd; c += blockDim.x) {
        const float v = __half2float(xr[c]);
        ss = fma((double)v, (double)v, ss);
    }
    const float inv = inv_rms(cta_sum(ss, part), 1.0 / (double)n_embd, eps);
    for (int c = threadIdx.x; c < n_embd; c += blockDim.x) {
        const float g = gamma ? __half2float(gamma[c]) : 1.0f;
        yr[c] = __float2half_rn(__fmul_rn(__fmul_rn(__half2float(xr[c]), inv), g));
    }
}

extern "C" __global__ void rope_rotate_half(const __half* x, const float* ctab, const float* stab, __half* y, int n_rows,
                                            int half_dim) {
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const __half* xr = x + (size_t)r * half_dim * 2;
    __half* yr = y + (size_t)r * half_dim * 2;
    const float* cr = ctab + (size_t)r * half_dim;
    const float* sr = stab + (size_t)r * half_dim;
    for (int i = threadIdx.x; i < half_dim; i += blockDim.x) {
        const float lo = __half2float(xr[i]), hi = __half2float(xr[i + half_dim]);
        const float c = cr[i], s = sr[i];
        yr[i] = __float2half_rn(__fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)));
        yr[i + half_dim] = __float2half_rn(__fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s)));
    }
}

