// moe_group.cuh -- groups a batch's (token, slot) entries by expert, the step that produces the expert-sorted row
// order the expert-tiled matmuls and the expert-grouped SwiGLU rows work in. Contract of the reference's moe_group
// (src/gpu_ops.hip:259-320, launcher src/gpu_ops.cpp:115-122): from ids [T][n_used] (expert of each slot),
//   tok_rows[i] = token and pair_rows[i] = token * n_used + slot of the i-th entry in expert order,
//   each expert's run cut into tiles of up to `tile` entries: tile_e / tile_start / tile_n, *n_tiles of them, in
//   expert order. Counts, run boundaries and tiles are deterministic.
// The reference leaves the order inside an expert's run to atomics; here it is fixed too (ascending pair index), so
// two runs give identical arrays: a thread owns a contiguous range of entries, per-range counts are scanned per
// expert, and every entry lands at (start of its expert's run) + (entries of that expert in earlier ranges) + (its
// rank inside its own range).
//
// One CTA of 1024 threads, as in the reference; n_expert <= 1024. Work memory: shared memory only (no scratch).
// The per-range, per-expert bookkeeping would need ranges x experts counters, so ranges are processed in rounds of
// 1024 entries (one entry per thread, in index order): a round ranks its entries with a warp match and a scan over
// the 32 warps, then advances the experts' running offsets. Cost is O(n / 1024) rounds; the reference's batches hold
// at most a few thousand tokens.

#ifndef B200_MOE_GROUP_CUH
#define B200_MOE_GROUP_CUH

#include "common.cuh"

namespace b200 {

#define MOE_MAX_EXPERTS 1024

__global__ void __launch_bounds__(1024)
k_moe_group(const int* ids, int T, int n_used, int n_expert, int tile, int* tok_rows, int* pair_rows, int* n_tiles,
            int* tile_e, int* tile_start, int* tile_n) {
    __shared__ int cnt[MOE_MAX_EXPERTS];    // entries per expert, then the next free entry of each expert's run
    __shared__ int wsum[2][32];
    __shared__ int round_cnt[MOE_MAX_EXPERTS];   // entries of each expert seen so far in the current round, by warp order
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int n = T * n_used;
    cnt[tid] = 0;
    round_cnt[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += 1024) {
        const int e = ids[i];
        if (e >= 0 && e < n_expert) atomicAdd(&cnt[e], 1);   // (integer counts: the order of the adds does not matter)
    }
    __syncthreads();
    // exclusive scans over the experts (thread e): entry offsets and tile offsets
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
        wsum[0][lane] = x - x0;   // exclusive bases per warp
        wsum[1][lane] = y - y0;
    }
    __syncthreads();
    const int eo = wsum[0][w] + a - c, to = wsum[1][w] + b - nt;
    __syncthreads();
    cnt[tid] = eo;   // the next free entry of expert tid's run
    if (tid < n_expert) {
        for (int k = 0; k < nt; ++k) {
            tile_e[to + k] = tid;
            tile_start[to + k] = eo + k * tile;
            tile_n[to + k] = min(tile, c - k * tile);
        }
        if (tid == n_expert - 1) *n_tiles = to + nt;
    }
    __syncthreads();
    // rounds of 1024 consecutive entries; inside a round warps take their turn in order, lanes rank by lane index
    for (int base = 0; base < n; base += 1024) {
        const int i = base + tid;
        const int e = i < n ? ids[i] : -1;
        const bool ok = e >= 0 && e < n_expert;
        const unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);   // lanes of this warp with my expert
        const int rank = __popc(peers & ((1u << lane) - 1u));                       // those before me
        const int mine = __popc(peers);
        const bool leader = ok && rank == 0;
        int before = 0;
        for (int turn = 0; turn < 32; ++turn) {   // warp `turn` claims its slots; later warps see its counts
            if (w == turn && leader) {
                before = round_cnt[e];
                round_cnt[e] = before + mine;
            }
            __syncthreads();
        }
        before = __shfl_sync(0xffffffffu, before, __ffs(peers) - 1);
        if (ok) {
            const int p = cnt[e] + before + rank;
            tok_rows[p] = i / n_used;
            pair_rows[p] = i;
        }
        __syncthreads();
        if (leader) {   // one lane per (warp, expert): fold this warp's share into the running offset
            atomicAdd(&cnt[e], mine);
        }
        __syncthreads();
        if (leader) round_cnt[e] = 0;
        __syncthreads();
    }
}

}  // namespace b200

#endif  // B200_MOE_GROUP_CUH
