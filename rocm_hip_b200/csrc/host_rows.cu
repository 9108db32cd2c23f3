// host_rows.cu -- the host-buffer entry points (part 3 of include/b200_layer_ops.h): rows that live in host memory are
// cut into chunks and streamed through copy-in -> kernel -> copy-out on a ring of staging slots, one stream per
// slot, so PCIe transfers in both directions overlap the kernels. This is the drop-in for callers of the reference's
// CPU functions (src/qwen_ops.h:17-48, the gather loop of src/qwen_model.cpp:980-986), which own host arrays.
// Rows are independent, so chunk boundaries never change a result: each row gets the bits the device launchers give.

#include "b200_layer_ops.h"

#include <string.h>

#include <new>
#include <vector>

struct b200_host_ctx {
    int device = 0;
    size_t slot_bytes = 0;
    std::vector<char*> slots;
    std::vector<cudaStream_t> streams;
    char* consts = nullptr;  // gammas, frequency factors, the bad-id flag
    cudaEvent_t consts_ready = nullptr;   // recorded after a call's constants were queued; every slot stream waits on it
};

namespace {

constexpr size_t kConstBytes = 1u << 20;
constexpr size_t kAlign = 256;
constexpr int kMaxBufs = 12;

inline size_t up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct RowBufs {
    const void* in[kMaxBufs];
    size_t in_bpr[kMaxBufs];
    int n_in = 0;
    void* out[kMaxBufs];
    size_t out_bpr[kMaxBufs];
    int n_out = 0;
    size_t tmp_bpr[kMaxBufs];   // rows that only live on the device between two kernels of a chunk
    int n_tmp = 0;
    int add_in(const void* p, size_t bpr) { in[n_in] = p; in_bpr[n_in] = bpr; return n_in++; }
    int add_out(void* p, size_t bpr) { out[n_out] = p; out_bpr[n_out] = bpr; return n_out++; }
    int add_tmp(size_t bpr) { tmp_bpr[n_tmp] = bpr; return n_tmp++; }
};

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// launch(dev_in, dev_out, rows, row0, stream[, dev_tmp]) -> cudaError_t
template <class F>
auto call_launch(F& launch, void** din, void** dout, void** dtmp, long long rows, long long row0, cudaStream_t st, int)
    -> decltype(launch(din, dout, rows, row0, st, dtmp)) {
    return launch(din, dout, rows, row0, st, dtmp);
}
template <class F>
cudaError_t call_launch(F& launch, void** din, void** dout, void**, long long rows, long long row0, cudaStream_t st, long) {
    return launch(din, dout, rows, row0, st);
}

// Chunk sizes for T rows through a ring of n_slots slots that hold cap rows each. The first chunk's copy in and the
// last chunk's copy out are not overlapped by anything, so the chunks start small (1/16 of a slot, at least 64 rows),
// double up to what a slot holds and halve again towards the end; in between, large chunks keep the count of copies
// and launches (a fixed cost of some tens of microseconds per chunk) low, but stay small enough for two chunks per
// slot when the work allows, so that the ring actually overlaps.
std::vector<long long> chunk_plan(long long T, long long cap, long long n_slots) {
    std::vector<long long> sizes;
    if (T <= 0 || cap <= 0 || n_slots <= 0) return sizes;
    const long long r0 = cap / 16 > 64 ? cap / 16 : (cap < 64 ? cap : 64);
    std::vector<long long> ramp;
    long long left = T, step = r0;
    while (step < cap && left > 4 * step) { ramp.push_back(step); left -= 2 * step; step *= 2; }
    long long mid = step < cap ? step : cap;
    const long long want = (left + 2 * n_slots - 1) / (2 * n_slots);
    if (mid > want && want >= 64) mid = want;
    sizes = ramp;
    for (; left > 0; left -= mid) sizes.push_back(left < mid ? left : mid);
    sizes.insert(sizes.end(), ramp.rbegin(), ramp.rend());
    return sizes;
}

template <class F>
cudaError_t run_rows(b200_host_ctx* ctx, long long T, const RowBufs& io, F launch) {
    size_t per_row = 0;
    for (int i = 0; i < io.n_in; ++i) per_row += io.in_bpr[i];
    for (int i = 0; i < io.n_out; ++i) per_row += io.out_bpr[i];
    for (int i = 0; i < io.n_tmp; ++i) per_row += io.tmp_bpr[i];
    const size_t slack = kAlign * (size_t)(io.n_in + io.n_out + io.n_tmp);
    if (per_row == 0 || ctx->slot_bytes <= slack || (ctx->slot_bytes - slack) / per_row == 0) return cudaErrorInvalidValue;
    const long long cap = (long long)((ctx->slot_bytes - slack) / per_row);   // rows a slot holds
    const std::vector<long long> sizes = chunk_plan(T, cap, (long long)ctx->slots.size());
    const long long chunk = cap;   // the slot's layout is that of its largest chunk
    cudaError_t err = cudaSuccess;
    long long row0 = 0;
    for (size_t c = 0; c < sizes.size() && err == cudaSuccess; row0 += sizes[c], ++c) {
        const long long rows = sizes[c];
        const size_t s = c % ctx->slots.size();
        cudaStream_t st = ctx->streams[s];
        char* base = ctx->slots[s];
        void* din[kMaxBufs];
        void* dout[kMaxBufs];
        void* dtmp[kMaxBufs];
        size_t off = 0;
        for (int i = 0; i < io.n_in; ++i) { din[i] = base + off; off += up((size_t)chunk * io.in_bpr[i]); }
        for (int i = 0; i < io.n_out; ++i) { dout[i] = base + off; off += up((size_t)chunk * io.out_bpr[i]); }
        for (int i = 0; i < io.n_tmp; ++i) { dtmp[i] = base + off; off += up((size_t)chunk * io.tmp_bpr[i]); }
        if (c < ctx->slots.size() && ctx->consts_ready) err = cudaStreamWaitEvent(st, ctx->consts_ready, 0);
        for (int i = 0; i < io.n_in && err == cudaSuccess; ++i)
            err = cudaMemcpyAsync(din[i], (const char*)io.in[i] + (size_t)row0 * io.in_bpr[i], (size_t)rows * io.in_bpr[i],
                                  cudaMemcpyHostToDevice, st);
        if (err == cudaSuccess) err = call_launch(launch, din, dout, dtmp, rows, row0, st, 0);
        for (int i = 0; i < io.n_out && err == cudaSuccess; ++i)
            err = cudaMemcpyAsync((char*)io.out[i] + (size_t)row0 * io.out_bpr[i], dout[i], (size_t)rows * io.out_bpr[i],
                                  cudaMemcpyDeviceToHost, st);
    }
    for (cudaStream_t st : ctx->streams) {
        const cudaError_t e = cudaStreamSynchronize(st);
        if (err == cudaSuccess) err = e;
    }
    return err;
}

// Copies small read-only arrays (gammas and the like) to the context's constant area before the chunks start: queued
// on the first slot's stream; done() records the event every slot stream waits on before its first chunk (the slot
// streams are non-blocking streams, which nothing else orders against these copies).
struct ConstArea {
    b200_host_ctx* ctx;
    size_t off = 0;
    cudaError_t err = cudaSuccess;
    explicit ConstArea(b200_host_ctx* c) : ctx(c) {}
    template <typename T>
    const T* put(const T* host, size_t count) {
        if (!host) return nullptr;
        const size_t bytes = count * sizeof(T);
        if (off + up(bytes) > kConstBytes) { err = cudaErrorInvalidValue; return nullptr; }
        char* d = ctx->consts + off;
        off += up(bytes);
        const cudaError_t e = cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, ctx->streams[0]);
        if (err == cudaSuccess) err = e;
        return reinterpret_cast<const T*>(d);
    }
    cudaError_t done() {
        if (err == cudaSuccess) err = cudaEventRecord(ctx->consts_ready, ctx->streams[0]);
        return err;
    }
};

}  // namespace

extern "C" {

int b200_host_chunk_plan(long long T, long long slot_rows, int n_slots, long long* sizes, int max_sizes) {
    const std::vector<long long> plan = chunk_plan(T, slot_rows, n_slots);
    for (size_t i = 0; i < plan.size() && (int)i < max_sizes; ++i) sizes[i] = plan[i];
    return (int)plan.size();
}

b200_host_ctx* b200_host_ctx_create(size_t slot_bytes, int n_slots) {
    if (slot_bytes < (1u << 16) || n_slots < 1 || n_slots > 16) return nullptr;
    b200_host_ctx* ctx = new (std::nothrow) b200_host_ctx;
    if (!ctx) return nullptr;
    ctx->slot_bytes = slot_bytes;
    bool ok = cudaGetDevice(&ctx->device) == cudaSuccess && gpu_ops_init("gpu_ops.co") == 0 &&
              cudaMalloc((void**)&ctx->consts, kConstBytes) == cudaSuccess;
    for (int i = 0; ok && i < n_slots; ++i) {
        char* p = nullptr;
        cudaStream_t st = nullptr;
        ok = cudaMalloc((void**)&p, slot_bytes) == cudaSuccess;
        if (ok) ctx->slots.push_back(p);
        ok = ok && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
        if (ok) ctx->streams.push_back(st);
    }
    ok = ok && cudaEventCreateWithFlags(&ctx->consts_ready, cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        b200_host_ctx_destroy(ctx);
        return nullptr;
    }
    return ctx;
}

void b200_host_ctx_destroy(b200_host_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard g(ctx->device);
    for (cudaStream_t st : ctx->streams) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
    for (char* p : ctx->slots) cudaFree(p);
    if (ctx->consts_ready) cudaEventDestroy(ctx->consts_ready);
    if (ctx->consts) cudaFree(ctx->consts);
    delete ctx;
}

cudaError_t b200_host_add_rmsnorm(b200_host_ctx* ctx, int elem, const void* x_in, const void* add, void* x_out,
                                  const float* w, void* y, int n, long long T, float eps) {
    if (!ctx || (elem != 2 && elem != 4) || !x_in || !y || n <= 0 || T <= 0 || (add && (!x_out || x_out == x_in)))
        return cudaErrorInvalidValue;
    DeviceGuard g(ctx->device);
    ConstArea ca(ctx);
    const float* dw = ca.put(w, (size_t)n);
    if (ca.done() != cudaSuccess) return ca.err;
    const size_t bpr = (size_t)n * elem;
    RowBufs io;
    io.add_in(x_in, bpr);
    if (add) { io.add_in(add, bpr); io.add_out(x_out, bpr); }
    io.add_out(y, bpr);
    const bool has_add = add != nullptr;
    return run_rows(ctx, T, io, [=](void** din, void** dout, long long rows, long long, cudaStream_t st) {
        void* dxo = has_add ? dout[0] : nullptr;
        void* dy = has_add ? dout[1] : dout[0];
        const void* da = has_add ? din[1] : nullptr;
        if (elem == 4)
            return gpu_add_rmsnorm_f32((const float*)din[0], (const float*)da, (float*)dxo, dw, (float*)dy, n, rows, eps, st);
        return gpu_add_rmsnorm_bf16((const uint16_t*)din[0], (const uint16_t*)da, (uint16_t*)dxo, dw, (uint16_t*)dy, n,
                                    rows, eps, st);
    });
}

cudaError_t b200_host_swiglu(b200_host_ctx* ctx, int elem, const void* g, const void* u, void* out, long long rows,
                             int width) {
    if (!ctx || (elem != 2 && elem != 4) || !g || !u || !out || rows <= 0 || width <= 0) return cudaErrorInvalidValue;
    DeviceGuard dg(ctx->device);
    const size_t bpr = (size_t)width * elem;
    RowBufs io;
    io.add_in(g, bpr);
    io.add_in(u, bpr);
    io.add_out(out, bpr);
    return run_rows(ctx, rows, io, [=](void** din, void** dout, long long r, long long, cudaStream_t st) {
        if (elem == 4) return gpu_swiglu_f32((const float*)din[0], (const float*)din[1], (float*)dout[0], r * width, st);
        return gpu_swiglu_bf16((const uint16_t*)din[0], (const uint16_t*)din[1], (uint16_t*)dout[0], r * width, st);
    });
}

cudaError_t b200_host_qk_norm_rope(b200_host_ctx* ctx, int elem, const void* qfull, const void* k, const float* q_norm,
                                   const float* k_norm, void* q_out, void* k_out, int n_q, int n_kv, int head_dim,
                                   int n_rot, int rot_pairs, const int* positions, int pos0, long long T,
                                   float freq_base, float eps, int gated, int qk_norm, const float* freq_factors) {
    if (!ctx || (elem != 2 && elem != 4) || T <= 0 || n_q < 0 || n_kv < 0 || n_q + n_kv <= 0 || head_dim <= 0 ||
        (n_q > 0 && (!qfull || !q_out)) || (n_kv > 0 && (!k || !k_out)) || n_rot < 0 || n_rot > head_dim)
        return cudaErrorInvalidValue;
    DeviceGuard dg(ctx->device);
    ConstArea ca(ctx);
    const float* dqn = ca.put(q_norm, (size_t)head_dim);
    const float* dkn = ca.put(k_norm, (size_t)head_dim);
    const float* dff = ca.put(freq_factors, (size_t)(n_rot / 2));
    if (ca.done() != cudaSuccess) return ca.err;
    const size_t qs = (size_t)(gated ? 2 * head_dim : head_dim);
    RowBufs io;
    int iq = -1, ik = -1, ip = -1, oq = -1, ok = -1;
    if (n_q > 0) { iq = io.n_in; io.add_in(qfull, (size_t)n_q * qs * elem); oq = io.n_out; io.add_out(q_out, (size_t)n_q * head_dim * elem); }
    if (n_kv > 0) { ik = io.n_in; io.add_in(k, (size_t)n_kv * head_dim * elem); ok = io.n_out; io.add_out(k_out, (size_t)n_kv * head_dim * elem); }
    if (positions) { ip = io.n_in; io.add_in(positions, sizeof(int)); }
    return run_rows(ctx, T, io, [=](void** din, void** dout, long long rows, long long row0, cudaStream_t st) {
        const void* dq = iq >= 0 ? din[iq] : nullptr;
        const void* dk = ik >= 0 ? din[ik] : nullptr;
        void* dqo = oq >= 0 ? dout[oq] : nullptr;
        void* dko = ok >= 0 ? dout[ok] : nullptr;
        const int* dp = ip >= 0 ? (const int*)din[ip] : nullptr;
        const int p0 = dp ? 0 : pos0 + (int)row0;
        if (elem == 4)
            return gpu_qk_norm_rope((const float*)dq, (const float*)dk, dqn, dkn, (float*)dqo, (float*)dko, n_q, n_kv,
                                    head_dim, n_rot, rot_pairs, dp, p0, rows, freq_base, eps, gated, qk_norm, dff, st);
        return gpu_qk_norm_rope_bf16((const uint16_t*)dq, (const uint16_t*)dk, dqn, dkn, (uint16_t*)dqo, (uint16_t*)dko,
                                     n_q, n_kv, head_dim, n_rot, rot_pairs, dp, p0, rows, freq_base, eps, gated, qk_norm,
                                     dff, st);
    });
}

cudaError_t b200_host_embed_rows(b200_host_ctx* ctx, int elem, int type, const void* table_dev, size_t row_bytes,
                                 int vocab, const int32_t* tokens, void* out, int E, long long T, float scale) {
    if (!ctx || (elem != 2 && elem != 4) || !table_dev || !tokens || !out || E <= 0 || T <= 0 || vocab <= 0)
        return cudaErrorInvalidValue;
    for (long long t = 0; t < T; ++t)  // the reference's range check, before any decode (src/qwen_model.cpp:981)
        if (tokens[t] < 0 || tokens[t] >= vocab) return cudaErrorInvalidValue;
    DeviceGuard dg(ctx->device);
    const int int_max = 0x7fffffff;
    ConstArea ca(ctx);
    int* flag = const_cast<int*>(ca.put(&int_max, 1));
    if (ca.done() != cudaSuccess) return ca.err;
    RowBufs io;
    io.add_in(tokens, sizeof(int32_t));
    io.add_out(out, (size_t)E * elem);
    return run_rows(ctx, T, io, [=](void** din, void** dout, long long rows, long long, cudaStream_t st) {
        if (elem == 4)
            return gpu_embed_rows(type, table_dev, row_bytes, vocab, (const int32_t*)din[0], (float*)dout[0], E, rows,
                                  scale, flag, st);
        return gpu_embed_rows_bf16(type, table_dev, row_bytes, vocab, (const int32_t*)din[0], (uint16_t*)dout[0], E, rows,
                                   scale, flag, st);
    });
}

cudaError_t b200_host_layer_sweep(b200_host_ctx* ctx, const b200_layer_sweep* a) {
    if (!ctx || !a || (a->elem != 2 && a->elem != 4) || a->T <= 0 || a->E <= 0 || a->FF <= 0 || a->vocab <= 0 ||
        !a->table_dev || !a->tokens || !a->xn_attn || !a->attn_proj || !a->xn_ffn || !a->gate || !a->up || !a->act ||
        !a->ffn_proj || !a->x_out || !a->xn_next || a->n_q < 0 || a->n_kv < 0 || a->head_dim <= 0 || a->n_rot < 0 ||
        a->n_rot > a->head_dim || (a->n_q > 0 && (!a->qfull || !a->q_out)) || (a->n_kv > 0 && (!a->k || !a->k_out)))
        return cudaErrorInvalidValue;
    for (long long t = 0; t < a->T; ++t)  // the reference's range check, before any decode (src/qwen_model.cpp:981)
        if (a->tokens[t] < 0 || a->tokens[t] >= a->vocab) return cudaErrorInvalidValue;
    DeviceGuard dg(ctx->device);
    const b200_layer_sweep s = *a;
    const int elem = s.elem, E = s.E, D = s.head_dim;
    const int int_max = 0x7fffffff;
    ConstArea ca(ctx);
    int* flag = const_cast<int*>(ca.put(&int_max, 1));
    const float* w1 = ca.put(s.w_attn_norm, (size_t)E);
    const float* w2 = ca.put(s.w_ffn_norm, (size_t)E);
    const float* w3 = ca.put(s.w_next_norm, (size_t)E);
    const float* dqn = ca.put(s.q_norm, (size_t)D);
    const float* dkn = ca.put(s.k_norm, (size_t)D);
    const float* dff = ca.put(s.freq_factors, (size_t)(s.n_rot / 2));
    if (ca.done() != cudaSuccess) return ca.err;
    const size_t row = (size_t)E * elem, qs = (size_t)(s.gated ? 2 * D : D);
    RowBufs io;
    const int i_tok = io.add_in(s.tokens, sizeof(int32_t));
    const int i_q = s.n_q > 0 ? io.add_in(s.qfull, (size_t)s.n_q * qs * elem) : -1;
    const int i_k = s.n_kv > 0 ? io.add_in(s.k, (size_t)s.n_kv * D * elem) : -1;
    const int i_pos = s.positions ? io.add_in(s.positions, sizeof(int)) : -1;
    const int i_p1 = io.add_in(s.attn_proj, row), i_g = io.add_in(s.gate, (size_t)s.FF * elem),
              i_u = io.add_in(s.up, (size_t)s.FF * elem), i_p2 = io.add_in(s.ffn_proj, row);
    const int o_xn1 = io.add_out(s.xn_attn, row);
    const int o_q = s.n_q > 0 ? io.add_out(s.q_out, (size_t)s.n_q * D * elem) : -1;
    const int o_k = s.n_kv > 0 ? io.add_out(s.k_out, (size_t)s.n_kv * D * elem) : -1;
    const int o_xn2 = io.add_out(s.xn_ffn, row), o_act = io.add_out(s.act, (size_t)s.FF * elem),
              o_x = io.add_out(s.x_out, row), o_xn3 = io.add_out(s.xn_next, row);
    const int t_x = io.add_tmp(row), t_alt = io.add_tmp(row);   // the residual stream between the kernels of a chunk
    return run_rows(ctx, s.T, io, [=](void** din, void** dout, long long rows, long long row0, cudaStream_t st, void** tmp) {
        const int* dp = i_pos >= 0 ? (const int*)din[i_pos] : nullptr;
        const int p0 = dp ? 0 : s.pos0 + (int)row0;
        cudaError_t e;
        if (elem == 4) {
            typedef float V;
            e = gpu_embed_rows(s.qtype, s.table_dev, s.row_bytes, s.vocab, (const int32_t*)din[i_tok], (V*)tmp[t_x], E, rows,
                               s.embd_scale, flag, st);
            if (e == cudaSuccess) e = gpu_add_rmsnorm_f32((const V*)tmp[t_x], nullptr, nullptr, w1, (V*)dout[o_xn1], E, rows, s.eps, st);
            if (e == cudaSuccess)
                e = gpu_qk_norm_rope(i_q >= 0 ? (const V*)din[i_q] : nullptr, i_k >= 0 ? (const V*)din[i_k] : nullptr, dqn, dkn,
                                     o_q >= 0 ? (V*)dout[o_q] : nullptr, o_k >= 0 ? (V*)dout[o_k] : nullptr, s.n_q, s.n_kv, D,
                                     s.n_rot, s.rot_pairs, dp, p0, rows, s.freq_base, s.eps, s.gated, s.qk_norm, dff, st);
            if (e == cudaSuccess)
                e = gpu_add_rmsnorm_f32((const V*)tmp[t_x], (const V*)din[i_p1], (V*)tmp[t_alt], w2, (V*)dout[o_xn2], E, rows, s.eps, st);
            if (e == cudaSuccess) e = gpu_swiglu_f32((const V*)din[i_g], (const V*)din[i_u], (V*)dout[o_act], rows * s.FF, st);
            if (e == cudaSuccess)
                e = gpu_add_rmsnorm_f32((const V*)tmp[t_alt], (const V*)din[i_p2], (V*)dout[o_x], w3, (V*)dout[o_xn3], E, rows, s.eps, st);
        } else {
            typedef uint16_t V;
            e = gpu_embed_rows_bf16(s.qtype, s.table_dev, s.row_bytes, s.vocab, (const int32_t*)din[i_tok], (V*)tmp[t_x], E,
                                    rows, s.embd_scale, flag, st);
            if (e == cudaSuccess) e = gpu_add_rmsnorm_bf16((const V*)tmp[t_x], nullptr, nullptr, w1, (V*)dout[o_xn1], E, rows, s.eps, st);
            if (e == cudaSuccess)
                e = gpu_qk_norm_rope_bf16(i_q >= 0 ? (const V*)din[i_q] : nullptr, i_k >= 0 ? (const V*)din[i_k] : nullptr, dqn,
                                          dkn, o_q >= 0 ? (V*)dout[o_q] : nullptr, o_k >= 0 ? (V*)dout[o_k] : nullptr, s.n_q,
                                          s.n_kv, D, s.n_rot, s.rot_pairs, dp, p0, rows, s.freq_base, s.eps, s.gated,
                                          s.qk_norm, dff, st);
            if (e == cudaSuccess)
                e = gpu_add_rmsnorm_bf16((const V*)tmp[t_x], (const V*)din[i_p1], (V*)tmp[t_alt], w2, (V*)dout[o_xn2], E, rows, s.eps, st);
            if (e == cudaSuccess) e = gpu_swiglu_bf16((const V*)din[i_g], (const V*)din[i_u], (V*)dout[o_act], rows * s.FF, st);
            if (e == cudaSuccess)
                e = gpu_add_rmsnorm_bf16((const V*)tmp[t_alt], (const V*)din[i_p2], (V*)dout[o_x], w3, (V*)dout[o_xn3], E, rows, s.eps, st);
        }
        return e;
    });
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Row sharding over several GPUs from ONE process: a group owns one host-buffer context per device; an operation
// cuts the rows into contiguous ranges (device g gets rows [T g / G, T (g + 1) / G)), and one host thread per device
// runs the single-device call on its range. Rows are independent, so nothing is exchanged between devices and each
// row gets the bits a single device would give it. Small read-only inputs (gammas, frequency factors) are copied to
// every device by the per-device call; the embedding table must already be resident on every device.

#include <thread>

struct b200_host_group {
    std::vector<b200_host_ctx*> ctx;
};

namespace {

template <class F>
cudaError_t for_each_device(b200_host_group* grp, long long T, F fn) {
    const int G = (int)grp->ctx.size();
    std::vector<cudaError_t> err((size_t)G, cudaSuccess);
    std::vector<std::thread> th;
    for (int g = 0; g < G; ++g) {
        const long long lo = T * g / G, hi = T * (g + 1) / G;
        if (hi <= lo) continue;
        th.emplace_back([&, g, lo, hi] { err[(size_t)g] = fn(grp->ctx[(size_t)g], g, lo, hi - lo); });
    }
    for (auto& t : th) t.join();
    for (cudaError_t e : err)
        if (e != cudaSuccess) return e;
    return cudaSuccess;
}

inline const char* at(const void* p, size_t bytes) { return p ? (const char*)p + bytes : nullptr; }
inline char* at(void* p, size_t bytes) { return p ? (char*)p + bytes : nullptr; }

}  // namespace

extern "C" {

b200_host_group* b200_host_group_create(int n_devices, size_t slot_bytes, int n_slots) {
    int have = 0;
    if (cudaGetDeviceCount(&have) != cudaSuccess || have < 1) return nullptr;
    if (n_devices <= 0) n_devices = have;
    if (n_devices > have) return nullptr;
    int prev = 0;
    (void)cudaGetDevice(&prev);
    b200_host_group* grp = new (std::nothrow) b200_host_group;
    if (!grp) return nullptr;
    for (int d = 0; d < n_devices; ++d) {
        b200_host_ctx* c = cudaSetDevice(d) == cudaSuccess ? b200_host_ctx_create(slot_bytes, n_slots) : nullptr;
        if (!c) {
            (void)cudaSetDevice(prev);
            b200_host_group_destroy(grp);
            return nullptr;
        }
        grp->ctx.push_back(c);
    }
    (void)cudaSetDevice(prev);
    return grp;
}

void b200_host_group_destroy(b200_host_group* grp) {
    if (!grp) return;
    for (b200_host_ctx* c : grp->ctx) b200_host_ctx_destroy(c);
    delete grp;
}

int b200_host_group_size(const b200_host_group* grp) { return grp ? (int)grp->ctx.size() : 0; }

cudaError_t b200_host_group_add_rmsnorm(b200_host_group* grp, int elem, const void* x_in, const void* add, void* x_out,
                                        const float* w, void* y, int n, long long T, float eps) {
    if (!grp || T <= 0 || n <= 0 || (elem != 2 && elem != 4)) return cudaErrorInvalidValue;
    const size_t bpr = (size_t)n * elem;
    return for_each_device(grp, T, [=](b200_host_ctx* c, int, long long lo, long long rows) {
        return b200_host_add_rmsnorm(c, elem, at(x_in, lo * bpr), at(add, lo * bpr), at(x_out, lo * bpr), w, at(y, lo * bpr), n,
                                     rows, eps);
    });
}

cudaError_t b200_host_group_swiglu(b200_host_group* grp, int elem, const void* g, const void* u, void* out, long long rows,
                                   int width) {
    if (!grp || rows <= 0 || width <= 0 || (elem != 2 && elem != 4)) return cudaErrorInvalidValue;
    const size_t bpr = (size_t)width * elem;
    return for_each_device(grp, rows, [=](b200_host_ctx* c, int, long long lo, long long r) {
        return b200_host_swiglu(c, elem, at(g, lo * bpr), at(u, lo * bpr), at(out, lo * bpr), r, width);
    });
}

cudaError_t b200_host_group_qk_norm_rope(b200_host_group* grp, int elem, const void* qfull, const void* k,
                                         const float* q_norm, const float* k_norm, void* q_out, void* k_out, int n_q,
                                         int n_kv, int head_dim, int n_rot, int rot_pairs, const int* positions, int pos0,
                                         long long T, float freq_base, float eps, int gated, int qk_norm,
                                         const float* freq_factors) {
    if (!grp || T <= 0 || head_dim <= 0 || (elem != 2 && elem != 4)) return cudaErrorInvalidValue;
    const size_t qi = (size_t)n_q * (gated ? 2 : 1) * head_dim * elem, qo = (size_t)n_q * head_dim * elem,
                 kb = (size_t)n_kv * head_dim * elem;
    return for_each_device(grp, T, [=](b200_host_ctx* c, int, long long lo, long long rows) {
        return b200_host_qk_norm_rope(c, elem, at(qfull, lo * qi), at(k, lo * kb), q_norm, k_norm, at(q_out, lo * qo),
                                      at(k_out, lo * kb), n_q, n_kv, head_dim, n_rot, rot_pairs,
                                      positions ? positions + lo : nullptr, positions ? 0 : pos0 + (int)lo, rows, freq_base,
                                      eps, gated, qk_norm, freq_factors);
    });
}

cudaError_t b200_host_group_embed_rows(b200_host_group* grp, int elem, int type, const void* const* tables_dev,
                                       size_t row_bytes, int vocab, const int32_t* tokens, void* out, int E, long long T,
                                       float scale) {
    if (!grp || !tables_dev || !tokens || T <= 0 || E <= 0 || (elem != 2 && elem != 4)) return cudaErrorInvalidValue;
    for (long long t = 0; t < T; ++t)   // refuse before any device starts (src/qwen_model.cpp:981)
        if (tokens[t] < 0 || tokens[t] >= vocab) return cudaErrorInvalidValue;
    const size_t bpr = (size_t)E * elem;
    return for_each_device(grp, T, [=](b200_host_ctx* c, int g, long long lo, long long rows) {
        return b200_host_embed_rows(c, elem, type, tables_dev[g], row_bytes, vocab, tokens + lo, at(out, lo * bpr), E, rows,
                                    scale);
    });
}

cudaError_t b200_host_group_layer_sweep(b200_host_group* grp, const b200_layer_sweep* a, const void* const* tables_dev) {
    if (!grp || !a || !tables_dev || a->T <= 0 || !a->tokens || (a->elem != 2 && a->elem != 4)) return cudaErrorInvalidValue;
    for (long long t = 0; t < a->T; ++t)   // refuse before any device starts (src/qwen_model.cpp:981)
        if (a->tokens[t] < 0 || a->tokens[t] >= a->vocab) return cudaErrorInvalidValue;
    const b200_layer_sweep all = *a;
    return for_each_device(grp, all.T, [=](b200_host_ctx* c, int g, long long lo, long long rows) {
        b200_layer_sweep s = all;
        const size_t e = (size_t)s.elem, row = (size_t)s.E * e, D = (size_t)s.head_dim;
        const size_t qin = (size_t)s.n_q * (s.gated ? 2 : 1) * D * e, kin = (size_t)s.n_kv * D * e, ff = (size_t)s.FF * e;
        s.T = rows;
        s.table_dev = tables_dev[g];
        s.tokens = all.tokens + lo;
        s.xn_attn = at(all.xn_attn, lo * row);
        s.qfull = at(all.qfull, lo * qin);
        s.k = at(all.k, lo * kin);
        s.q_out = at(all.q_out, lo * (size_t)s.n_q * D * e);
        s.k_out = at(all.k_out, lo * kin);
        if (all.positions) s.positions = all.positions + lo;
        else s.pos0 = all.pos0 + (int)lo;
        s.attn_proj = at(all.attn_proj, lo * row);
        s.xn_ffn = at(all.xn_ffn, lo * row);
        s.gate = at(all.gate, lo * ff);
        s.up = at(all.up, lo * ff);
        s.act = at(all.act, lo * ff);
        s.ffn_proj = at(all.ffn_proj, lo * row);
        s.x_out = at(all.x_out, lo * row);
        s.xn_next = at(all.xn_next, lo * row);
        return b200_host_layer_sweep(c, &s);
    });
}

}  // extern "C"
