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
// k_moe_group: one CTA of 1024 threads, as in the reference; n_expert <= 1024. Work memory: shared memory only.
// The per-range, per-expert bookkeeping would need ranges x experts counters, so ranges are processed in rounds of
// 1024 entries (one entry per thread, in index order): a round ranks its entries with a warp match and a scan over
// the 32 warps, then advances the experts' running offsets. Cost is O(n / 1024) rounds: right for the reference's
// batches of a few thousand tokens; longer batches take the segment kernels at the end of this file.

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

// ---------------------------------------------------------------------------------------------------------------
// Long batches: the same result (bit for bit the arrays k_moe_group writes) from three launches that use the whole
// device. The n entries are cut into segments of seg_len consecutive entries (a multiple of 32), one warp each:
//   k_moe_seg_count    counts [seg][expert]: entries of each expert in each segment (shared-memory histogram per warp)
//   k_moe_seg_scan     one CTA, thread e: run start of expert e (scan of the totals), the tiles, and counts [seg][e]
//                      turned into the position of segment seg's first entry of expert e
//   k_moe_seg_scatter  each warp walks its segment in index order, 32 entries per step, ranks the lanes of one expert
//                      with a warp match and places them at the running position of that expert
// Work memory: n_segs * n_expert ints of device scratch. A warp's shared-memory counters are touched by that warp
// alone, so __syncwarp is the only synchronisation inside a segment.

#define MOE_SEG_WARPS 8   // warps (segments) per CTA

__device__ __forceinline__ void moe_zero_row(int* row, int n_expert, int lane) {
    for (int e = lane; e < n_expert; e += 32) row[e] = 0;
    __syncwarp();
}

__global__ void __launch_bounds__(32 * MOE_SEG_WARPS)
k_moe_seg_count(const int* ids, int n, int n_expert, int seg_len, int n_segs, int* counts) {
    __shared__ int hist[MOE_SEG_WARPS][MOE_MAX_EXPERTS];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int seg = blockIdx.x * MOE_SEG_WARPS + w;
    if (seg >= n_segs) return;
    int* h = hist[w];
    moe_zero_row(h, n_expert, lane);
    const long long lo = (long long)seg * seg_len, hi = min((long long)n, lo + seg_len);   // (n may be near INT_MAX)
    for (long long base = lo; base < hi; base += 32) {
        const long long i = base + lane;
        const int e = i < hi ? ids[i] : -1;
        const bool ok = e >= 0 && e < n_expert;
        const unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
        if (ok && (peers & ((1u << lane) - 1u)) == 0) h[e] += __popc(peers);   // one lane per expert present
        __syncwarp();
    }
    for (int e = lane; e < n_expert; e += 32) counts[(size_t)seg * n_expert + e] = h[e];
}

// ep: n_expert rounded up to a power of two. The 1024 threads are 1024 / ep parts x ep experts: a part sums and
// later rewrites a contiguous range of segments, so small expert counts still keep every thread busy.
__global__ void __launch_bounds__(1024)
k_moe_seg_scan(int n_expert, int ep, int tile, int n_segs, int* counts, int* n_tiles, int* tile_e, int* tile_start,
               int* tile_n) {
    __shared__ int wsum[2][32];
    __shared__ int psum[1024];
    __shared__ int estart[MOE_MAX_EXPERTS];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int parts = 1024 / ep, e = tid & (ep - 1), part = tid / ep;
    const int per = (n_segs + parts - 1) / parts, s0 = part * per, s1 = min(n_segs, s0 + per);
    int mine = 0;
    if (e < n_expert)
        for (int s = s0; s < s1; ++s) mine += counts[(size_t)s * n_expert + e];
    psum[tid] = mine;
    __syncthreads();
    int c = 0;   // thread tid < n_expert: the total of expert tid
    if (tid < n_expert)
        for (int p = 0; p < parts; ++p) c += psum[p * ep + tid];
    const int nt = (c + tile - 1) / tile;
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
    if (tid < n_expert) {
        estart[tid] = eo;
        for (int k = 0; k < nt; ++k) {
            tile_e[to + k] = tid;
            tile_start[to + k] = eo + k * tile;
            tile_n[to + k] = min(tile, c - k * tile);
        }
        if (tid == n_expert - 1) *n_tiles = to + nt;
    }
    __syncthreads();
    if (e < n_expert) {
        int run = estart[e];
        for (int p = 0; p < part; ++p) run += psum[p * ep + e];
        for (int s = s0; s < s1; ++s) {
            int* q = counts + (size_t)s * n_expert + e;
            const int v = *q;
            *q = run;
            run += v;
        }
    }
}

__global__ void __launch_bounds__(32 * MOE_SEG_WARPS)
k_moe_seg_scatter(const int* ids, int n, int n_used, int n_expert, int seg_len, int n_segs, const int* offsets,
                  int* tok_rows, int* pair_rows) {
    __shared__ int next[MOE_SEG_WARPS][MOE_MAX_EXPERTS];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int seg = blockIdx.x * MOE_SEG_WARPS + w;
    if (seg >= n_segs) return;
    int* nx = next[w];
    for (int e = lane; e < n_expert; e += 32) nx[e] = offsets[(size_t)seg * n_expert + e];
    __syncwarp();
    const long long lo = (long long)seg * seg_len, hi = min((long long)n, lo + seg_len);
    for (long long base = lo; base < hi; base += 32) {
        const long long i = base + lane;
        const int e = i < hi ? ids[i] : -1;
        const bool ok = e >= 0 && e < n_expert;
        const unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        int p = 0;
        if (ok) p = nx[e] + rank;
        __syncwarp();
        if (ok && rank == 0) nx[e] += __popc(peers);
        __syncwarp();
        if (ok) {
            tok_rows[p] = (int)(i / n_used);
            pair_rows[p] = (int)i;
        }
    }
}

}  // namespace b200

#endif  // B200_MOE_GROUP_CUH
