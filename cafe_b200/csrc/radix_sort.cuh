// radix_sort.cuh -- stable LSD radix sort of (key, position) pairs on sm_100a, written for this library's
// three sorts: lookups by main-table bucket, lookups by LRU-table bucket (the order in which the sequential
// insert of tricks/sketch.cpp:268-296 meets the ids of one bucket must be kept, hence stable), and the
// scatter's lookups by table row.  Keys are bucket or row numbers of 17 to 20 bits, so two passes of up to
// 10 bits do; a pass is two small kernels and one scatter:
//   k_rs_hist         digit histogram of every tile of CAFE_RS_TILE keys            -> hist[digit][tile]
//   k_rs_scan_cols    per digit, exclusive prefix over the tiles (in place)         -> totals[digit]
//   k_rs_scatter      every key to (totals of the digits before its own) + hist[digit][tile] + its rank among the tile's keys of
//                     that digit, ranks taken in index order (warp match + per-warp counters), so equal
//                     keys keep their order
// The first pass can take its keys straight from the ids (hash of the id into nb buckets), and the last
// pass can also write the ids in sorted order, so that the replay kernels stream them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "sketch_core.cuh"

#define CAFE_RS_THREADS 256
#define CAFE_RS_ITEMS 8
#define CAFE_RS_TILE (CAFE_RS_THREADS * CAFE_RS_ITEMS)
#define CAFE_RS_MAX_BITS 10
#define CAFE_RS_MAX_BINS (1 << CAFE_RS_MAX_BITS)
#define CAFE_RS_WARPS (CAFE_RS_THREADS / 32)

struct CafeKeySource {
    const uint32_t* key;   // explicit keys, or (null) ...
    const uint32_t* gid;   // ... ids hashed into nb buckets
    int32_t nb;
};
__device__ __forceinline__ uint32_t cafe_rs_key(const CafeKeySource& S, int64_t i) {
    return S.key ? S.key[i] : (uint32_t)cafe_hash(S.gid[i], S.nb);
}

static inline int cafe_rs_tiles(int64_t n) { return (int)((n + CAFE_RS_TILE - 1) / CAFE_RS_TILE); }
// scratch of one sort of at most `cap` pairs, in int32 elements: hist[bins][tiles] followed by totals[bins]
static inline size_t cafe_rs_scratch_elems(int64_t cap) { return (size_t)CAFE_RS_MAX_BINS * (size_t)(cafe_rs_tiles(cap) + 1); }

static __global__ void __launch_bounds__(CAFE_RS_THREADS)
k_rs_hist(const CafeKeySource S, int n, int shift, int bits, int32_t* __restrict__ hist, int tiles) {
    __shared__ int s_cnt[CAFE_RS_MAX_BINS];
    const int bins = 1 << bits;
    for (int d = threadIdx.x; d < bins; d += CAFE_RS_THREADS) s_cnt[d] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * CAFE_RS_TILE;
#pragma unroll 4
    for (int it = 0; it < CAFE_RS_ITEMS; ++it) {
        const int64_t i = base + it * CAFE_RS_THREADS + threadIdx.x;
        if (i < n) atomicAdd(&s_cnt[(cafe_rs_key(S, i) >> shift) & (bins - 1)], 1);
    }
    __syncthreads();
    for (int d = threadIdx.x; d < bins; d += CAFE_RS_THREADS) hist[(size_t)d * tiles + blockIdx.x] = s_cnt[d];
}

// exclusive prefix of v over the block's threads, and the block total
__device__ __forceinline__ int cafe_rs_block_exclusive(int v, int* total, int* s_warp) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
    }
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    int before = 0, all = 0;
    for (int q = 0; q < nw; ++q) { const int t = s_warp[q]; if (q < w) before += t; all += t; }
    __syncthreads();
    *total = all;
    return before + inc - v;
}

// one block per digit: exclusive prefix over the tiles, in place; totals[digit] = sum
static __global__ void __launch_bounds__(CAFE_RS_THREADS)
k_rs_scan_cols(int32_t* __restrict__ hist, int tiles, int32_t* __restrict__ totals) {
    __shared__ int s_warp[CAFE_RS_WARPS];
    int32_t* col = hist + (size_t)blockIdx.x * tiles;
    int run = 0;
    for (int t0 = 0; t0 < tiles; t0 += CAFE_RS_THREADS) {
        const int t = t0 + threadIdx.x;
        const int v = t < tiles ? col[t] : 0;
        int tot;
        const int ex = cafe_rs_block_exclusive(v, &tot, s_warp);
        if (t < tiles) col[t] = run + ex;
        run += tot;
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = run;
}

// val_in == null: the value of pair i is i.  gather_src != null: gather_out[sorted index] = gather_src[value].
static __global__ void __launch_bounds__(CAFE_RS_THREADS)
k_rs_scatter(const CafeKeySource S, const int32_t* __restrict__ val_in, uint32_t* __restrict__ key_out,
             int32_t* __restrict__ val_out, int n, int shift, int bits, const int32_t* __restrict__ hist, int tiles,
             const int32_t* __restrict__ totals, const uint32_t* __restrict__ gather_src, uint32_t* __restrict__ gather_out) {
    __shared__ int s_hist[CAFE_RS_WARPS][CAFE_RS_MAX_BINS];   // per warp: keys of each digit seen so far, then the prefix over warps
    __shared__ int s_base[CAFE_RS_MAX_BINS];                  // first output index of the tile's keys of each digit
    __shared__ int s_warp[CAFE_RS_WARPS];
    const int bins = 1 << bits;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int d = threadIdx.x; d < bins; d += CAFE_RS_THREADS) {
#pragma unroll
        for (int q = 0; q < CAFE_RS_WARPS; ++q) s_hist[q][d] = 0;
    }
    {
        // first output index of every digit = the digits' totals before it (every block adds them up itself: at most
        // 1024 numbers, which saves a launch per pass) + the tile's place among the tiles' keys of that digit
        constexpr int PER = CAFE_RS_MAX_BINS / CAFE_RS_THREADS;
        int loc[PER], sum = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = (int)threadIdx.x * PER + i;
            loc[i] = d < bins ? totals[d] : 0;
            sum += loc[i];
        }
        int tot;
        int ex = cafe_rs_block_exclusive(sum, &tot, s_warp);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = (int)threadIdx.x * PER + i;
            if (d < bins) s_base[d] = ex + hist[(size_t)d * tiles + blockIdx.x];
            ex += loc[i];
        }
    }
    __syncthreads();
    // a warp owns CAFE_RS_ITEMS * 32 consecutive pairs and walks them 32 at a time, so (iteration, lane) is index order
    const int64_t base = (int64_t)blockIdx.x * CAFE_RS_TILE + (int64_t)w * (32 * CAFE_RS_ITEMS);
    uint32_t key[CAFE_RS_ITEMS];
    int32_t val[CAFE_RS_ITEMS];
    int32_t rank[CAFE_RS_ITEMS];
#pragma unroll
    for (int it = 0; it < CAFE_RS_ITEMS; ++it) {
        const int64_t i = base + it * 32 + lane;
        key[it] = i < n ? cafe_rs_key(S, i) : 0u;
        val[it] = i < n ? (val_in ? val_in[i] : (int32_t)i) : 0;
    }
#pragma unroll
    for (int it = 0; it < CAFE_RS_ITEMS; ++it) {
        const int64_t i = base + it * 32 + lane;
        const bool ok = i < n;
        const int d = (int)((key[it] >> shift) & (uint32_t)(bins - 1));
        // lanes beyond the end take digits of their own so that they match nobody
        const unsigned peers = __match_any_sync(0xffffffffu, ok ? d : bins + lane);
        const int ahead = __popc(peers & ((1u << lane) - 1u));
        const int before = ok ? s_hist[w][d] : 0;
        __syncwarp();
        if (ok && ahead == 0) s_hist[w][d] = before + __popc(peers);
        __syncwarp();
        rank[it] = before + ahead;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < bins; d += CAFE_RS_THREADS) {
        int run = 0;
#pragma unroll
        for (int q = 0; q < CAFE_RS_WARPS; ++q) { const int t = s_hist[q][d]; s_hist[q][d] = run; run += t; }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < CAFE_RS_ITEMS; ++it) {
        const int64_t i = base + it * 32 + lane;
        if (i >= n) continue;
        const int d = (int)((key[it] >> shift) & (uint32_t)(bins - 1));
        const int64_t o = (int64_t)s_base[d] + s_hist[w][d] + rank[it];
        key_out[o] = key[it];
        val_out[o] = val[it];
        if (gather_src) gather_out[o] = gather_src[val[it]];
    }
}

// Sorts n pairs by the low `total_bits` bits of their keys, stably.  The sorted pairs end in (key_out, val_out);
// (key_tmp, val_tmp) hold the intermediate pass and must not alias anything else.  scratch: cafe_rs_scratch_elems(n)
// int32 elements.  Returns the first launch error, if any.
static inline cudaError_t cafe_radix_sort(const CafeKeySource& src, const int32_t* val_in, uint32_t* key_tmp, int32_t* val_tmp,
                                          uint32_t* key_out, int32_t* val_out, int n, int total_bits, int32_t* scratch,
                                          const uint32_t* gather_src, uint32_t* gather_out, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    if (total_bits < 1) total_bits = 1;
    const int passes = (total_bits + CAFE_RS_MAX_BITS - 1) / CAFE_RS_MAX_BITS;
    const int bits = (total_bits + passes - 1) / passes;
    const int tiles = cafe_rs_tiles(n);
    int32_t* hist = scratch;
    int32_t* totals = scratch + (size_t)CAFE_RS_MAX_BINS * tiles;
    CafeKeySource S = src;
    const int32_t* vin = val_in;
    for (int p = 0; p < passes; ++p) {
        const bool last = p == passes - 1;
        // ping-pong so that the last pass lands in the output arrays
        const bool to_out = ((passes - 1 - p) & 1) == 0;
        uint32_t* ko = to_out ? key_out : key_tmp;
        int32_t* vo = to_out ? val_out : val_tmp;
        const int shift = p * bits;
        k_rs_hist<<<tiles, CAFE_RS_THREADS, 0, st>>>(S, n, shift, bits, hist, tiles);
        k_rs_scan_cols<<<1 << bits, CAFE_RS_THREADS, 0, st>>>(hist, tiles, totals);
        k_rs_scatter<<<tiles, CAFE_RS_THREADS, 0, st>>>(S, vin, ko, vo, n, shift, bits, hist, tiles, totals,
                                                         last ? gather_src : nullptr, last ? gather_out : nullptr);
        S.key = ko; S.gid = nullptr; S.nb = 0;
        vin = vo;
    }
    return cudaGetLastError();
}
