// embed.cuh -- token-embedding gather and dequantisation from a GGUF Q8_0 / Q4_0 table resident in HBM, the B200
// kernel behind gpu_embed_rows. It replaces the reference's single-threaded host loop (src/qwen_model.cpp:980-986:
// range check, then qt_to_float of row tokens[t] into output row t) and restates its block decoders bit for bit
// (src/quant_types.cpp:181-189 Q8_0: y = qs[j] * d; :78-91 Q4_0: value j from the low nibble of qs[j], value j + 16
// from the high nibble, each (nibble - 8) * d; d widened exactly from fp16). One fp32 multiply per value, nothing
// fused with it; an embedding scale other than 1 is a second, separately rounded multiply (src/qwen_model.cpp:1409).
//
// Layout: table rows of E / 32 blocks (34 or 18 bytes each), row t at table + t * row_bytes; inside a row the fp16
// scale and the payload are only 2-byte aligned. A warp copies a row (or a slice of one) into its own shared-memory
// slice, then decodes from shared memory so that every global store is a full 16-byte vector and a warp writes 512
// contiguous bytes. Traffic per token: 4 (id) + row_bytes + E * s_out, the algorithmic minimum.
// Three kernels share the decoder (embed_decode_chunk): k_embed_rows_sliced (long batches: a warp per 1.4 KB slice,
// one slice per warp, CTAs retiring in slice order), k_embed_rows_bulk (short batches: a resident grid whose warps
// keep four slices in flight as bulk copies), k_embed_rows (any alignment and E % 32 == 0: whole row per warp,
// 16-byte loads when the table base and row_bytes allow, else 2-byte loads). The launcher picks by shape and length.
// An id outside [0, vocab) never touches the table: its output row is zero-filled and the smallest offending row
// index is recorded in *bad_row (initialised to INT_MAX by the launcher's caller) for the host to turn into an error.

#ifndef B200_EMBED_CUH
#define B200_EMBED_CUH

#include "common.cuh"

namespace b200 {

#define B200_QT_Q4_0 2
#define B200_QT_Q8_0 8

// Rows are staged in chunks of at most EMBED_CHUNK_BLOCKS blocks (a multiple of 8 so that chunk starts keep the
// row's 16-byte alignment: 8 * 34 and 8 * 18 are multiples of 16).
#define EMBED_CHUNK_BLOCKS 160
#define EMBED_WARPS 8

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// N (4 or 8) consecutive bytes starting at the 2-byte aligned shared-memory address p, as N / 4 little-endian words:
// aligned 32-bit loads from the word that holds p's first byte and a funnel shift by the 0 or 16 bits p sits into
// it (the last load may reach up to 4 bytes past p + N: the stage buffers are padded for it).
template <int N>
__device__ __forceinline__ void ld_bytes_2al(const uint8_t* p, uint32_t* w) {
    const unsigned a = smem_u32(p), base = a & ~3u, sh = (a & 2u) << 3;
    uint32_t r[N / 4 + 1];
#pragma unroll
    for (int i = 0; i <= N / 4; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r[i]) : "r"(base + 4 * i));
#pragma unroll
    for (int i = 0; i < N / 4; ++i) w[i] = __funnelshift_r(r[i], r[i + 1], sh);
}

// Bytes k and k + 1 of w, each an unsigned integer below 256, as the exact floats 2^23 + byte (the byte dropped into
// the low mantissa bits of 0x4B000000): subtracting 2^23 + bias then gives the signed integer as a float with no
// rounding and without the int-to-float conversion unit, whose rate (a quarter of the fp32 rate) bounded this kernel.
__device__ __forceinline__ f2 bytes_to_magic(uint32_t w, int k) {
    const uint32_t m = 0x4B000000u;
    return pk2(__uint_as_float(__byte_perm(w, m, 0x7650 + k)), __uint_as_float(__byte_perm(w, m, 0x7651 + k)));
}

// Decodes the cb blocks staged at sm (block b at sm + b * BB) into o (the row's values from the chunk's first block
// on): per step a lane takes VPL consecutive values of one block and stores them as one 16-byte vector, so a warp
// step writes 512 contiguous bytes. Bit for bit (float)q * d (then * scale): the integer is formed exactly, the
// products are separately rounded two-wide multiplies.
template <typename OUT, int TYPE>
__device__ __forceinline__ void embed_decode_chunk(const uint8_t* sm, int cb, OUT* o_chunk, float scale, int lane) {
    constexpr int BB = TYPE == B200_QT_Q8_0 ? 34 : 18;            // bytes per block
    constexpr int VPL = sizeof(OUT) == 4 ? 4 : 8;                 // values per lane and step: one 16-byte store
    constexpr int LPB = 32 / VPL;                                 // lanes per block
    constexpr int BPS = 32 / LPB;                                 // blocks per warp step
    const int sub = lane % LPB;
    const f2 scale2 = pk2(scale, scale);
    for (int bs = 0; bs < cb; bs += BPS) {
        const int b = bs + lane / LPB;
        if (b < cb) {
            const uint8_t* blk = sm + b * BB;
            const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
            const f2 d2 = pk2(d, d);
            f2 y[VPL / 2];
            if constexpr (TYPE == B200_QT_Q8_0) {
                // int8 q as the unsigned byte q + 128: 2^23 + 128 + q, minus 2^23 + 128
                const f2 off = pk2(8388736.0f, 8388736.0f);
                uint32_t w[VPL / 4];
                ld_bytes_2al<VPL>(blk + 2 + sub * VPL, w);
#pragma unroll
                for (int i = 0; i < VPL / 4; ++i) {
                    const uint32_t x = w[i] ^ 0x80808080u;
                    y[2 * i] = mul2(sub2(bytes_to_magic(x, 0), off), d2);
                    y[2 * i + 1] = mul2(sub2(bytes_to_magic(x, 2), off), d2);
                }
            } else {
                // values [sub * VPL, sub * VPL + VPL) of the block: the first 16 are low nibbles, the rest high;
                // nibble - 8 from 2^23 + nibble minus 2^23 + 8
                const f2 off = pk2(8388616.0f, 8388616.0f);
                const int v0 = sub * VPL, byte0 = v0 & 15, shift = v0 < 16 ? 0 : 4;
                uint32_t w[VPL / 4];
                ld_bytes_2al<VPL>(blk + 2 + byte0, w);
#pragma unroll
                for (int i = 0; i < VPL / 4; ++i) {
                    const uint32_t x = (w[i] >> shift) & 0x0F0F0F0Fu;
                    y[2 * i] = mul2(sub2(bytes_to_magic(x, 0), off), d2);
                    y[2 * i + 1] = mul2(sub2(bytes_to_magic(x, 2), off), d2);
                }
            }
            if (scale != 1.0f) {
#pragma unroll
                for (int i = 0; i < VPL / 2; ++i) y[i] = mul2(y[i], scale2);
            }
            OUT* o = o_chunk + (size_t)b * 32 + sub * VPL;
            if constexpr (sizeof(OUT) == 4) st_stream(o, Io2<float>::pack(y));
            else st_stream(o, Io2<__nv_bfloat16>::pack(y));
        }
    }
}

template <typename OUT, int TYPE>
__global__ void __launch_bounds__(EMBED_WARPS * 32)
k_embed_rows(const uint8_t* table, size_t row_bytes, int vocab, const int32_t* tokens, OUT* out, int E, long long T,
             float scale, int* bad_row, int vec_ok) {
    pdl_entry();
    constexpr int BB = TYPE == B200_QT_Q8_0 ? 34 : 18;            // bytes per block
    constexpr int VPL = sizeof(OUT) == 4 ? 4 : 8;                 // values per lane and 16-byte store
    __shared__ __align__(16) uint8_t stage[EMBED_WARPS][EMBED_CHUNK_BLOCKS * BB + 16];   // (+16: see ld_bytes_2al)
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint8_t* sm = stage[wid];
    const int nb = E / 32;
    const long long warp0 = (long long)blockIdx.x * EMBED_WARPS + wid, nwarps = (long long)gridDim.x * EMBED_WARPS;

    for (long long t = warp0; t < T; t += nwarps) {
        const int tok = tokens[t];
        OUT* orow = out + (size_t)t * E;
        if (tok < 0 || tok >= vocab) {
            if (lane == 0) atomicMin(bad_row, (int)(t < 0x7fffffff ? t : 0x7ffffffe));
            for (int c = lane * VPL; c < E; c += 32 * VPL) st_stream(orow + c, make_uint4(0, 0, 0, 0));
            continue;
        }
        const uint8_t* src = table + (size_t)tok * row_bytes;
        for (int b0 = 0; b0 < nb; b0 += EMBED_CHUNK_BLOCKS) {
            const int cb = min(EMBED_CHUNK_BLOCKS, nb - b0), bytes = cb * BB;
            const uint8_t* s = src + (size_t)b0 * BB;
            __syncwarp();  // the previous chunk has been decoded
            if (vec_ok) {
                const int nv = bytes >> 4;
                for (int i = lane; i < nv; i += 32) reinterpret_cast<uint4*>(sm)[i] = ld_stream(s + (size_t)i * 16);
                for (int i = (nv << 4) + lane * 2; i < bytes; i += 64)  // a chunk that is not a whole number of vectors
                    *reinterpret_cast<uint16_t*>(sm + i) = *reinterpret_cast<const uint16_t*>(s + i);
            } else {
                for (int i = lane * 2; i < bytes; i += 64)
                    *reinterpret_cast<uint16_t*>(sm + i) = *reinterpret_cast<const uint16_t*>(s + i);
            }
            __syncwarp();
            embed_decode_chunk<OUT, TYPE>(sm, cb, orow + (size_t)b0 * 32, scale, lane);
        }
    }
}

// The same load -> decode loop with a finer work unit: a warp takes one SLICE of a row (EMBED_SLICE_BYTES of blocks)
// at a time, and consecutive warps take consecutive slices, so that the warps running at any moment read and write a
// window of memory several times smaller than with a whole row per warp.
#define EMBED_SLICE_BYTES 1440

template <typename OUT, int TYPE>
__global__ void __launch_bounds__(EMBED_WARPS * 32)
k_embed_rows_sliced(const uint8_t* table, size_t row_bytes, int vocab, const int32_t* tokens, OUT* out, int E, long long T,
                    float scale, int* bad_row) {
    pdl_entry();
    constexpr int BB = TYPE == B200_QT_Q8_0 ? 34 : 18;
    constexpr int VPL = sizeof(OUT) == 4 ? 4 : 8;
    constexpr int SB = EMBED_SLICE_BYTES / BB / 8 * 8;   // blocks per slice, a multiple of 8 (slices stay 16-byte aligned)
    __shared__ __align__(16) uint8_t stage[EMBED_WARPS][SB * BB + 16];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint8_t* sm = stage[wid];
    const int nb = E / 32, S = (nb + SB - 1) / SB;
    const long long warp0 = (long long)blockIdx.x * EMBED_WARPS + wid, nwarps = (long long)gridDim.x * EMBED_WARPS;
    const long long total = T * S;
    const bool small = total <= 0xffffffffLL;   // (uniform) the slice index fits 32 bits: a 32-bit division finds its row
    for (long long i = warp0; i < total; i += nwarps) {
        long long t;
        int si;
        if (small) {
            const unsigned iu = (unsigned)i, tu = iu / (unsigned)S;
            t = tu;
            si = (int)(iu - tu * (unsigned)S);
        } else {
            t = i / S;
            si = (int)(i - t * S);
        }
        const int b0 = si * SB, cb = min(SB, nb - b0);
        const int tok = tokens[t];
        OUT* o = out + (size_t)t * E + (size_t)b0 * 32;
        if (tok < 0 || tok >= vocab) {
            if (lane == 0 && b0 == 0) atomicMin(bad_row, (int)(t < 0x7fffffff ? t : 0x7ffffffe));
            for (int c = lane * VPL; c < cb * 32; c += 32 * VPL) st_stream(o + c, make_uint4(0, 0, 0, 0));
            continue;
        }
        const uint8_t* s = table + (size_t)tok * row_bytes + (size_t)b0 * BB;
        const int nv = (cb * BB) >> 4;   // whole 16-byte vectors: cb is a multiple of 8
        __syncwarp();  // the previous slice has been decoded
        for (int v = lane; v < nv; v += 32) reinterpret_cast<uint4*>(sm)[v] = ld_stream(s + (size_t)v * 16);
        __syncwarp();
        embed_decode_chunk<OUT, TYPE>(sm, cb, o, scale, lane);
    }
}

// The same gather with the row fetch overlapped with the decode. A warp owns EMBED_BULK_SLOTS shared-memory slices of
// about 1.4 KB each and walks its tokens' rows slice by slice: while it decodes one slice, the bulk copies
// of the next EMBED_BULK_SLOTS - 1 (one instruction each, issued by lane 0, completion counted on the slice's mbarrier)
// are under way, so a warp always has HBM requests in flight and never idles between "row requested" and "row arrived"
// as the load -> decode loop of k_embed_rows does. The ids of the warp's next 64 tokens are fetched 32 at a time, one
// per lane, so that no copy waits for an id load first. Needs a 16-byte aligned table, row_bytes % 16 == 0 and rows of
// whole 8-block groups (E % 256 == 0: every slice is then a multiple of 16 bytes).
// A wait that runs out of polls (never seen; it would mean a lost copy) records -1 in *bad_row and the warp stops.
#define EMBED_BULK_WARPS 8
#define EMBED_BULK_SLICE_BYTES 1440   // payload of a slice: 40 Q8_0 blocks (a quarter of a 5120-wide row) or 80 Q4_0 blocks
#define EMBED_BULK_SLOTS 4

template <typename OUT, int TYPE>
__global__ void __launch_bounds__(EMBED_BULK_WARPS * 32)
k_embed_rows_bulk(const uint8_t* table, size_t row_bytes, int vocab, const int32_t* tokens, OUT* out, int E, long long T,
                  float scale, int* bad_row) {
    pdl_entry();
    constexpr int BB = TYPE == B200_QT_Q8_0 ? 34 : 18;
    constexpr int VPL = sizeof(OUT) == 4 ? 4 : 8;
    constexpr int NS = EMBED_BULK_SLOTS;
    constexpr int SB = EMBED_BULK_SLICE_BYTES / BB / 8 * 8;   // blocks per slice, a multiple of 8
    constexpr int SLOT = SB * BB + 16;                        // a multiple of 16 (+16: see ld_bytes_2al)
    __shared__ __align__(128) uint8_t stage[EMBED_BULK_WARPS][NS][SLOT];
    __shared__ __align__(8) unsigned long long bar[EMBED_BULK_WARPS][NS];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nb = E / 32, nchunks = (nb + SB - 1) / SB;
    const long long warp0 = (long long)blockIdx.x * EMBED_BULK_WARPS + wid, nwarps = (long long)gridDim.x * EMBED_BULK_WARPS;
    if (lane < NS) mbar_init(&bar[wid][lane], 1);
    if (lane == 0) mbar_fence_init();
    __syncwarp();
    if (warp0 >= T) return;
    const long long ntok = (T - warp0 + nwarps - 1) / nwarps;   // this warp's tokens: warp0 + k * nwarps, k < ntok
    // ids of tokens k in [kb, kb + 32) (cur) and [kb + 32, kb + 64) (nxt), lane j holding the j-th
    long long kb = 0;
    auto load_ids = [&](long long k0) { return k0 + lane < ntok ? __ldg(tokens + warp0 + (k0 + lane) * nwarps) : 0; };
    int cur = load_ids(0), nxt = load_ids(32);
    auto id_of = [&](long long k) {   // every lane calls it with the same k in [kb, kb + 64)
        const int a = __shfl_sync(0xffffffffu, cur, (int)(k - kb) & 31), b = __shfl_sync(0xffffffffu, nxt, (int)(k - kb) & 31);
        return k - kb < 32 ? a : b;
    };
    auto start_copy = [&](int tok, int c, int slot) {   // lane 0 only, tok in range
        const int b0 = c * SB, cb = min(SB, nb - b0);
        fence_async_smem();
        bulk_g2s(stage[wid][slot], table + (size_t)tok * row_bytes + (size_t)b0 * BB, (unsigned)(cb * BB), &bar[wid][slot]);
    };
    // issue cursor (ik, ic, islot): the next slice to request; it runs NS - 1 slices ahead of the decode cursor
    long long ik = 0;
    int ic = 0, islot = 0;
    auto issue_one = [&]() {   // all lanes (the id comes by shuffle); no-op past the end
        if (ik >= ntok) return;
        const int tok = id_of(ik);
        if (lane == 0 && tok >= 0 && tok < vocab) start_copy(tok, ic, islot);
        islot = islot + 1 == NS ? 0 : islot + 1;
        if (++ic == nchunks) { ic = 0; ++ik; }
    };
#pragma unroll
    for (int i = 0; i < NS - 1; ++i) issue_one();
    unsigned phases = 0u;   // bit s: the parity slice s is waited for next
    int slot = 0;
    for (long long k = 0; k < ntok; ++k) {
        if (k - kb >= 32) {   // the decode cursor leaves the first id batch (the issue cursor is at most a few tokens ahead)
            kb += 32;
            cur = nxt;
            nxt = load_ids(kb + 32);
        }
        const long long t = warp0 + k * nwarps;
        const int tok = id_of(k);
        const bool valid = tok >= 0 && tok < vocab;
        OUT* orow = out + (size_t)t * E;
        if (!valid) {
            if (lane == 0) atomicMin(bad_row, (int)(t < 0x7fffffff ? t : 0x7ffffffe));
            for (int c = lane * VPL; c < E; c += 32 * VPL) st_stream(orow + c, make_uint4(0, 0, 0, 0));
        }
        for (int c = 0; c < nchunks; ++c) {
            // the slice decoded in the previous iteration (a __syncwarp ago) is free: request the slice NS - 1 ahead into it
            issue_one();
            const int s_now = slot;
            slot = slot + 1 == NS ? 0 : slot + 1;
            if (!valid) continue;
            const int b0 = c * SB, cb = min(SB, nb - b0);
            // lane 0 polls; the others learn the outcome by shuffle (a warp-wide poll multiplies the shared-memory traffic)
            int arrived = lane == 0 ? (int)mbar_wait(&bar[wid][s_now], (phases >> s_now) & 1u) : 0;
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            if (!arrived) {
                if (lane == 0) atomicMin(bad_row, -1);
                // (the other slices' copies, if in flight, get the same bounded wait before the slices go away)
                for (int o = 0; o < NS; ++o)
                    if (o != s_now) (void)mbar_wait(&bar[wid][o], (phases >> o) & 1u);
                return;
            }
            phases ^= 1u << s_now;
            embed_decode_chunk<OUT, TYPE>(stage[wid][s_now], cb, orow + (size_t)b0 * 32, scale, lane);
            __syncwarp();   // every lane has read the slice
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The other row formats a GGUF token_embd.weight comes in (src/quant_types.cpp:58-74 plain, :126-179 Q4_1 / Q5_0 /
// Q5_1, :264-345 Q4_K / Q5_K / Q6_K), decoded value for value as the reference's qt_to_float does, each product, sum
// and difference rounded on its own. Same shape as k_embed_rows: a warp per token, the row staged in the warp's
// shared-memory slice in chunks of whole blocks, a lane decoding runs of VPL consecutive values (a run never leaves
// a 16-value group, so one set of block constants serves it) and storing one 16-byte vector per run.

#define B200_QT_F32 0
#define B200_QT_F16 1
#define B200_QT_Q4_1 3
#define B200_QT_Q5_0 6
#define B200_QT_Q5_1 7
#define B200_QT_Q4_K 12
#define B200_QT_Q5_K 13
#define B200_QT_Q6_K 14
#define B200_QT_BF16 30

template <int TYPE>
struct RowFormat {   // BLK values in BB bytes; plain types are taken 32 values at a time
    static constexpr int BLK = (TYPE == B200_QT_Q4_K || TYPE == B200_QT_Q5_K || TYPE == B200_QT_Q6_K) ? 256 : 32;
    static constexpr int BB = TYPE == B200_QT_F32 ? 128 : (TYPE == B200_QT_F16 || TYPE == B200_QT_BF16) ? 64
                            : TYPE == B200_QT_Q4_1 ? 20 : TYPE == B200_QT_Q5_0 ? 22 : TYPE == B200_QT_Q5_1 ? 24
                            : TYPE == B200_QT_Q4_K ? 144 : TYPE == B200_QT_Q5_K ? 176 : TYPE == B200_QT_Q6_K ? 210
                            : TYPE == B200_QT_Q8_0 ? 34 : 18;
    // blocks per staged chunk: as many as fit the warp's slice, a count whose bytes are a multiple of 16
    static constexpr int GRAIN = BB % 16 == 0 ? 1 : BB % 8 == 0 ? 2 : BB % 4 == 0 ? 4 : 8;
    static constexpr int CHUNK = (EMBED_CHUNK_BLOCKS * 34 / BB) / GRAIN * GRAIN;
};

__device__ __forceinline__ float sm_f16(const uint8_t* p) { return f16_bits_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

// The 6-bit scale and minimum j of a K-quant super-block's 12 packed bytes (src/quant_types.cpp:192-200)
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// N (4 or 8) consecutive bytes at p as one little-endian word, fetched with the widest shared-memory loads that the
// alignment A (a power of two that divides p's offset in the stage buffer) allows
template <int N, int A>
__device__ __forceinline__ uint64_t ld_bytes(const uint8_t* p) {
    if constexpr (A >= 8 && N == 8) {
        return *reinterpret_cast<const uint64_t*>(p);
    } else if constexpr (A >= 4) {
        uint64_t w = *reinterpret_cast<const uint32_t*>(p);
        if constexpr (N == 8) w |= (uint64_t)*reinterpret_cast<const uint32_t*>(p + 4) << 32;
        return w;
    } else {
        uint64_t w = 0;
#pragma unroll
        for (int k = 0; k < N / 2; ++k) w |= (uint64_t)*reinterpret_cast<const uint16_t*>(p + 2 * k) << (16 * k);
        return w;
    }
}

// Values j0 .. j0 + N - 1 of the block at blk (N = 4 or 8, j0 a multiple of N). Block starts are multiples of
// gcd(BB, 16) bytes in the stage buffer, which fixes the alignment of every field below.
template <int TYPE, int N>
__device__ __forceinline__ void decode_run(const uint8_t* blk, int j0, float* y) {
    if constexpr (TYPE == B200_QT_F32) {
#pragma unroll
        for (int k = 0; k < N; ++k) y[k] = __uint_as_float(*reinterpret_cast<const uint32_t*>(blk + 4 * (j0 + k)));
    } else if constexpr (TYPE == B200_QT_F16) {
#pragma unroll
        for (int k = 0; k < N; ++k) y[k] = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 2 * (j0 + k)));
    } else if constexpr (TYPE == B200_QT_BF16) {
#pragma unroll
        for (int k = 0; k < N; ++k)
            y[k] = __uint_as_float((uint32_t)*reinterpret_cast<const uint16_t*>(blk + 2 * (j0 + k)) << 16);
    } else if constexpr (TYPE == B200_QT_Q4_1) {
        const float d = sm_f16(blk), m = sm_f16(blk + 2);
        const uint64_t qs = ld_bytes<N, 4>(blk + 4 + (j0 & 15)) >> (j0 < 16 ? 0 : 4);
#pragma unroll
        for (int k = 0; k < N; ++k) y[k] = __fadd_rn(__fmul_rn((float)((uint32_t)(qs >> (8 * k)) & 15u), d), m);
    } else if constexpr (TYPE == B200_QT_Q5_0 || TYPE == B200_QT_Q5_1) {
        constexpr bool ONE = TYPE == B200_QT_Q5_1;
        const float d = sm_f16(blk), m = ONE ? sm_f16(blk + 2) : 0.0f;
        const uint8_t* hb = blk + (ONE ? 4 : 2);
        const uint32_t qh = hb[0] | (hb[1] << 8) | (hb[2] << 16) | ((uint32_t)hb[3] << 24);
        const uint64_t qs = ld_bytes<N, ONE ? 8 : 2>(blk + (ONE ? 8 : 6) + (j0 & 15)) >> (j0 < 16 ? 0 : 4);
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const int x = (int)((uint32_t)(qs >> (8 * k)) & 15u) | (int)(((qh >> (j0 + k)) & 1u) << 4);   // bit j of qh: value j's fifth bit
            y[k] = ONE ? __fadd_rn(__fmul_rn((float)x, d), m) : __fmul_rn((float)(x - 16), d);
        }
    } else if constexpr (TYPE == B200_QT_Q4_K || TYPE == B200_QT_Q5_K) {
        constexpr bool FIVE = TYPE == B200_QT_Q5_K;
        const float d = sm_f16(blk), dmin = sm_f16(blk + 2);
        const int g = j0 >> 6, half = (j0 >> 5) & 1, l0 = j0 & 31;
        int sc, mn;
        k4_scale_min(2 * g + half, blk + 4, sc, mn);
        const float dd = __fmul_rn(d, (float)sc), mm = __fmul_rn(dmin, (float)mn);
        const uint64_t ql = ld_bytes<N, 8>(blk + (FIVE ? 48 : 16) + g * 32 + l0) >> (half ? 4 : 0);
        const uint64_t qh = FIVE ? ld_bytes<N, 8>(blk + 16 + l0) >> (2 * g + half) : 0;
#pragma unroll
        for (int k = 0; k < N; ++k) {
            int v = (int)((uint32_t)(ql >> (8 * k)) & 15u);
            if (FIVE) v += (int)((uint32_t)(qh >> (8 * k)) & 1u) << 4;
            y[k] = __fsub_rn(__fmul_rn(dd, (float)v), mm);
        }
    } else if constexpr (TYPE == B200_QT_Q6_K) {
        const float d = sm_f16(blk + 208);
        const int h = j0 >> 7, quarter = (j0 >> 5) & 3, l0 = j0 & 31;
        const uint64_t ql = ld_bytes<N, 2>(blk + h * 64 + l0 + ((quarter & 1) ? 32 : 0)) >> (quarter < 2 ? 0 : 4);
        const uint64_t qh = ld_bytes<N, 2>(blk + 128 + h * 32 + l0) >> (2 * quarter);
        const float ds = __fmul_rn(d, (float)(int8_t)blk[192 + h * 8 + (l0 >> 4) + 2 * quarter]);
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const int q = (int)(((uint32_t)(ql >> (8 * k)) & 15u) | (((uint32_t)(qh >> (8 * k)) & 3u) << 4)) - 32;
            y[k] = __fmul_rn(ds, (float)q);
        }
    }
}

template <typename OUT, int TYPE>
__global__ void __launch_bounds__(EMBED_WARPS * 32)
k_embed_rows_any(const uint8_t* table, size_t row_bytes, int vocab, const int32_t* tokens, OUT* out, int E, long long T,
                 float scale, int* bad_row, int vec_ok) {
    pdl_entry();
    using F = RowFormat<TYPE>;
    constexpr int VPL = sizeof(OUT) == 4 ? 4 : 8;
    __shared__ __align__(16) uint8_t stage[EMBED_WARPS][EMBED_CHUNK_BLOCKS * 34];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint8_t* sm = stage[wid];
    const int nb = E / F::BLK;
    const long long warp0 = (long long)blockIdx.x * EMBED_WARPS + wid, nwarps = (long long)gridDim.x * EMBED_WARPS;
    for (long long t = warp0; t < T; t += nwarps) {
        const int tok = tokens[t];
        OUT* orow = out + (size_t)t * E;
        if (tok < 0 || tok >= vocab) {
            if (lane == 0) atomicMin(bad_row, (int)(t < 0x7fffffff ? t : 0x7ffffffe));
            for (int c = lane * VPL; c < E; c += 32 * VPL) st_stream(orow + c, make_uint4(0, 0, 0, 0));
            continue;
        }
        const uint8_t* src = table + (size_t)tok * row_bytes;
        for (int b0 = 0; b0 < nb; b0 += F::CHUNK) {
            const int cb = min(F::CHUNK, nb - b0), bytes = cb * F::BB;
            const uint8_t* s = src + (size_t)b0 * F::BB;
            __syncwarp();
            if (vec_ok) {
                const int nv = bytes >> 4;
                for (int i = lane; i < nv; i += 32) reinterpret_cast<uint4*>(sm)[i] = ld_stream(s + (size_t)i * 16);
                for (int i = (nv << 4) + lane * 2; i < bytes; i += 64)
                    *reinterpret_cast<uint16_t*>(sm + i) = *reinterpret_cast<const uint16_t*>(s + i);
            } else {
                for (int i = lane * 2; i < bytes; i += 64)
                    *reinterpret_cast<uint16_t*>(sm + i) = *reinterpret_cast<const uint16_t*>(s + i);
            }
            __syncwarp();
            for (int v = lane * VPL; v < cb * F::BLK; v += 32 * VPL) {
                const int b = v / F::BLK, j0 = v % F::BLK;
                float y[VPL];
                decode_run<TYPE, VPL>(sm + b * F::BB, j0, y);
                if (scale != 1.0f) {
#pragma unroll
                    for (int k = 0; k < VPL; ++k) y[k] = __fmul_rn(y[k], scale);
                }
                OUT* o = orow + (size_t)(b0 + b) * F::BLK + j0;
                if constexpr (sizeof(OUT) == 4) {
                    st_stream(o, make_uint4(__float_as_uint(y[0]), __float_as_uint(y[1]), __float_as_uint(y[2]),
                                            __float_as_uint(y[3])));
                } else {
                    st_stream(o, make_uint4(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]),
                                            pack_bf16(y[6], y[7])));
                }
            }
        }
    }
}

}  // namespace b200

#endif  // B200_EMBED_CUH
