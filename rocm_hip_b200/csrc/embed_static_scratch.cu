// embed_static_scratch.cu -- gpu_embed_rows_static_scratch: the embedding gather for callers that must not allocate.
//
// Some hosts of this library cannot give a launcher device memory at call time. An inference engine that sizes all
// of HBM once at start-up (weights, KV cache, activation scratch) has nothing left to hand out later, and a serving
// loop usually forbids cudaMalloc outright because it can stall every stream of the device. The ordinary host-id
// entry point (gpu_embed_rows_host_ids) asks such a caller for a device buffer to hold the token ids and a device
// flag for bad ids; this one brings both with it, in a fixed array that is part of the library image.
//
// The price is a fixed ceiling and a shared buffer:
//   * at most B200_STATIC_SCRATCH_MAX_IDS ids per call (one MiB of ids; every GPU that loads the library carries the
//     array until the process exits);
//   * every call on a device writes the same array, so two calls whose GPU work can overlap (different streams,
//     different threads) race on it: keep calls on one stream, or order them yourself;
//   * the array keeps whatever the previous call left: each call overwrites the ids it needs and resets the flag
//     word before launching, nothing else is assumed clean.
// The first call on each device looks up the array's device address (cudaGetSymbolAddress), once.

#include "b200_layer_ops.h"

#include <mutex>

#include "embed.cuh"
#include "internal.h"

using namespace b200;

#define B200_STATIC_SCRATCH_MAX_IDS 262144

// [0, MAX_IDS): the ids of the current call; [MAX_IDS]: the kernel's bad-id flag (the rest of the tail pads to 256 B)
static __device__ __align__(256) int32_t g_id_scratch[B200_STATIC_SCRATCH_MAX_IDS + 64];

namespace {

constexpr int kMaxDevices = 64;
int32_t* g_scratch_addr[kMaxDevices];   // device address of g_id_scratch per device; in host code the symbol itself
bool g_scratch_known[kMaxDevices];      // is only a stand-in and must never be handed to a kernel
std::mutex g_setup_lock;

// Device address of the scratch array on the current device, looked up once per device
cudaError_t scratch_address(int32_t** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_scratch_known[dev]) {
        int32_t* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_id_scratch);
        if (e != cudaSuccess) return e;
        if (!p) return cudaErrorInvalidSymbol;
        g_scratch_addr[dev] = p;
        g_scratch_known[dev] = true;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

template <int TYPE>
cudaError_t launch(const uint8_t* table, size_t row_bytes, int vocab, const int32_t* ids_dev, float* out, int E,
                   long long T, float scale, int* flag_dev, int vec_ok, cudaStream_t stream) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_embed_rows<float, TYPE>, EMBED_WARPS * 32, 0);
    if (e != cudaSuccess) return e;
    const long long need = (T + EMBED_WARPS - 1) / EMBED_WARPS, resident = (long long)(per_sm > 0 ? per_sm : 1) * sms;
    k_embed_rows<float, TYPE><<<(unsigned)(need < resident ? need : resident), EMBED_WARPS * 32, 0, stream>>>(
        table, row_bytes, vocab, ids_dev, out, E, T, scale, flag_dev, vec_ok);
    return launched();
}

}  // namespace

extern "C" cudaError_t gpu_embed_rows_static_scratch(int type, const void* table, size_t row_bytes, int vocab,
                                                     const int32_t* tokens_host, float* out, int E, long long T,
                                                     float scale, cudaStream_t stream) {
    if (!lib_ready()) return cudaErrorInvalidDeviceFunction;   // before gpu_ops_init, as every launcher
    // Q8_0 and Q4_0 tables only (the formats the gather is built and measured for; the other row formats go through
    // gpu_embed_rows_host_ids with caller-owned scratch)
    const size_t bb = type == B200_QT_Q8_0 ? 34 : type == B200_QT_Q4_0 ? 18 : 0;
    if (!bb || !table || !tokens_host || !out || T <= 0 || E <= 0 || E % 32 != 0 || vocab <= 0 ||
        row_bytes < (size_t)(E / 32) * bb || row_bytes % 2 != 0 || (reinterpret_cast<uintptr_t>(table) & 1u) ||
        (reinterpret_cast<uintptr_t>(out) & 15u))
        return cudaErrorInvalidValue;
    if (T > B200_STATIC_SCRATCH_MAX_IDS) return cudaErrorInvalidValue;   // more ids than the built-in scratch holds
    for (long long t = 0; t < T; ++t)   // the reference's range check, before anything is queued (src/qwen_model.cpp:981)
        if (tokens_host[t] < 0 || tokens_host[t] >= vocab) return cudaErrorInvalidValue;

    int32_t* scratch = nullptr;
    cudaError_t e = scratch_address(&scratch);
    if (e != cudaSuccess) return e;
    int* flag = scratch + B200_STATIC_SCRATCH_MAX_IDS;
    // the array still holds the previous call's ids and flag: overwrite the T ids this call reads, and put the flag
    // word back to a value above every row index (0x7f7f7f7f) so that the kernel's atomicMin starts fresh
    e = cudaMemcpyAsync(scratch, tokens_host, (size_t)T * sizeof(int32_t), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(flag, 0x7f, sizeof(int), stream);
    if (e != cudaSuccess) return e;
    const int vec_ok = (reinterpret_cast<uintptr_t>(table) & 15u) == 0 && row_bytes % 16 == 0;
    const uint8_t* tb = static_cast<const uint8_t*>(table);
    return type == B200_QT_Q8_0
               ? launch<B200_QT_Q8_0>(tb, row_bytes, vocab, scratch, out, E, T, scale, flag, vec_ok, stream)
               : launch<B200_QT_Q4_0>(tb, row_bytes, vocab, scratch, out, E, T, scale, flag, vec_ok, stream);
}
