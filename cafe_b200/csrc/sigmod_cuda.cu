// sigmod_cuda.cu -- the one-stage HotSketch of the reference's artifact tree on sm_100a.
//
// Reference being replaced: class SS of ArtifactEvaluation/embeddings/sketch.cpp (the sketch of the SIGMOD'24
// CAFE paper): `lim` buckets of four slots kept sorted by count (Insert :89-123), Space-Saving replacement of the
// last slot, a FIFO of free hot rows, a multiplicative decay of every count once the inserted mass exceeds
// 10 * lim * k (decay :76-88, checked at the head of batch_insert(_val) :131-149), query (:43-51) and the
// free-list rebuild after a checkpoint load (update :61-75).  The reference keeps one such sketch per field
// (ss[26], :151); here every sketch is a handle.
//
// Parallel insert.  Within one call the FIFO is only popped (rows come back at decay time, which is a call
// boundary), so it stays non-empty up to its q_size-th successful pop and is empty from then on.  Lookups are
// sorted by (bucket, position) with the library's stable radix sort and every bucket is replayed twice:
//   pass A  assumes every candidate pop succeeds and flags the candidates (an id is a candidate at its first
//           lookup that finds its count at or above the threshold without a row);
//   scan    numbers the candidates in position order;
//   pass B  replays again: candidate number r takes row ring[q_head + r] if r < q_size and fails otherwise.
// Before the first failure in a bucket the two replays are identical, and every candidate behind a failure
// (flagged or new) lies behind the q_size-th success and fails too, so pass B is the sequential result.
// All scalars (inserted mass, FIFO head and size, rows handed out) live in device memory: a call queues a fixed
// sequence of kernels and never synchronises; the decay kernels return at once when no decay is due.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/cafe_b200.h"
#include "cafe_internal.h"
#include "radix_sort.cuh"

#define SG_TPB 256
#define SG_BLK 1024   // buckets (resp. positions) per block of the ordered-prefix kernels

struct alignas(16) SgBucket {   // 48 B (sketch.cpp:17-21)
    uint32_t val[4];
    float cnt[4];
    int32_t dic[4];
};
struct SgState {   // device-resident scalars of one sketch
    double tot;          // inserted mass since the last decay (sketch.cpp:13, 90)
    uint32_t q_head;
    int32_t q_size;
    int32_t num;         // rows handed out so far (:100)
    int32_t need_decay;
    int32_t n_cand;      // candidates of the call in flight
    int32_t decays;
    int32_t pad[2];
};
struct SgHandle {
    int lim = 0, k = 0, cap = 0, device = 0;
    double dr = 0.99;
    uint32_t ring_mask = 0;
    SgBucket* b = nullptr;
    uint32_t* ring = nullptr;
    SgState* st = nullptr;
    uint32_t *key = nullptr, *key_tmp = nullptr, *skey = nullptr, *sgid = nullptr;
    int32_t *pos_tmp = nullptr, *ord = nullptr, *start = nullptr, *rank = nullptr, *blk = nullptr, *sort_scratch = nullptr;
    float* simp = nullptr;
    uint8_t* cand = nullptr;
    double* partial = nullptr;
};

static inline int sg_blocks(int64_t n, int per = SG_TPB) { return (int)((n + per - 1) / per); }

__device__ __forceinline__ int sg_block_exclusive(int v, int* total, int* s_warp) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
    }
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int q = 0; q < SG_TPB / 32; ++q) { const int t = s_warp[q]; if (q < w) before += t; all += t; }
    __syncthreads();
    *total = all;
    return before + inc - v;
}
// sum of blk[0 .. blockIdx.x) (every block adds up its predecessors' counts itself)
__device__ __forceinline__ int sg_blocks_before(const int32_t* blk, int* s_warp) {
    int v = 0;
    for (int q = threadIdx.x; q < (int)blockIdx.x; q += SG_TPB) v += blk[q];
    int tot;
    sg_block_exclusive(v, &tot, s_warp);
    return tot;
}

__global__ void k_sg_iota(uint32_t* p, int n, uint32_t first) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = first + (uint32_t)i;
}

// ---- query (sketch.cpp:43-51): -row if the id sits in its bucket with a row, else the id -----------------
__device__ __forceinline__ int32_t sg_probe(const SgBucket* __restrict__ tb, int s, uint32_t x) {
    const SgBucket* b = &tb[x % (uint32_t)s];
    const uint4 v = *reinterpret_cast<const uint4*>(b->val);
    const float4 c = *reinterpret_cast<const float4*>(b->cnt);
    const int4 d = *reinterpret_cast<const int4*>(b->dic);
    // the first slot that holds the id decides (slots are scanned in order, :45-49)
    if (c.x != 0.f && v.x == x) return d.x;
    if (c.y != 0.f && v.y == x) return d.y;
    if (c.z != 0.f && v.z == x) return d.z;
    if (c.w != 0.f && v.w == x) return d.w;
    return 0;
}
__global__ void k_sg_query(const SgBucket* __restrict__ tb, int s, const uint32_t* __restrict__ gid, int n, int32_t* __restrict__ out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t x = gid[i];
    const int32_t r = sg_probe(tb, s, x);
    out[i] = r ? -r : (int32_t)x;
}
// ids of one field -> global ids and row codes (-hot row, or global id % hash_size), as cafe_embed_resolve does
template <typename IdT>
__global__ void k_sg_resolve(const SgBucket* __restrict__ tb, int s, const IdT* __restrict__ ids, int64_t f_offset, int hash_size,
                             int n, uint32_t* __restrict__ gid_out, int32_t* __restrict__ row_out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t x = (uint32_t)((int64_t)ids[i] + f_offset);
    const int32_t r = sg_probe(tb, s, x);
    gid_out[i] = x;
    row_out[i] = r ? -r : (int32_t)(x % (uint32_t)hash_size);
}
// hot row of every lookup that was handed one (insert result 1), for the migration (sk_embedding_bag.py:173-180)
__global__ void k_sg_post_rows(const SgBucket* __restrict__ tb, int s, const uint32_t* __restrict__ gid, const int32_t* __restrict__ mask,
                               int n, int32_t* __restrict__ out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = mask[i] ? sg_probe(tb, s, gid[i]) : 0;
}

// ---- decay (sketch.cpp:76-88), only when the call boundary test says so ----------------------------------
__global__ void k_sg_begin(SgState* st, int s, int k) {
    st->need_decay = st->tot > (double)(1ll * s * k * 10) ? 1 : 0;   // :132, :141
    st->n_cand = 0;
}
__device__ __forceinline__ bool sg_loses_row(float cnt, int32_t dic, double dr, int k) {
    return dic != 0 && (double)cnt * dr < (double)k;   // :79
}
__global__ void __launch_bounds__(SG_TPB) k_sg_decay_count(const SgBucket* __restrict__ tb, int s, const SgState* st, double dr, int k,
                                                           int32_t* __restrict__ blk) {
    __shared__ int s_warp[SG_TPB / 32];
    if (!st->need_decay) return;
    int c = 0;
    for (int q = 0; q < SG_BLK / SG_TPB; ++q) {
        const int key = blockIdx.x * SG_BLK + threadIdx.x * (SG_BLK / SG_TPB) + q;
        if (key < s) {
            const SgBucket b = tb[key];
#pragma unroll
            for (int i = 0; i < 4; ++i) c += sg_loses_row(b.cnt[i], b.dic[i], dr, k) ? 1 : 0;
        }
    }
    int tot;
    sg_block_exclusive(c, &tot, s_warp);
    if (threadIdx.x == 0) blk[blockIdx.x] = tot;
}
// rows go back to the FIFO in bucket order, slot order (the order of the reference's loop), then every count decays
__global__ void __launch_bounds__(SG_TPB) k_sg_decay_apply(SgBucket* __restrict__ tb, int s, const SgState* st, double dr, int k,
                                                           const int32_t* __restrict__ blk, uint32_t* __restrict__ ring, uint32_t mask) {
    __shared__ int s_warp[SG_TPB / 32];
    if (!st->need_decay) return;
    const int base = sg_blocks_before(blk, s_warp);
    constexpr int PER = SG_BLK / SG_TPB;
    SgBucket b[PER];
    int c = 0;
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        const int key = blockIdx.x * SG_BLK + threadIdx.x * PER + q;
        if (key < s) {
            b[q] = tb[key];
#pragma unroll
            for (int i = 0; i < 4; ++i) c += sg_loses_row(b[q].cnt[i], b[q].dic[i], dr, k) ? 1 : 0;
        }
    }
    int tot;
    int j = base + sg_block_exclusive(c, &tot, s_warp);
    const uint32_t tail = st->q_head + (uint32_t)st->q_size;
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        const int key = blockIdx.x * SG_BLK + threadIdx.x * PER + q;
        if (key >= s) break;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (sg_loses_row(b[q].cnt[i], b[q].dic[i], dr, k)) { ring[(tail + (uint32_t)j++) & mask] = (uint32_t)b[q].dic[i]; b[q].dic[i] = 0; }
            b[q].cnt[i] = (float)((double)b[q].cnt[i] * dr);   // :83 (float *= double)
        }
        tb[key] = b[q];
    }
}
__global__ void k_sg_decay_end(SgState* st, const int32_t* __restrict__ blk, int nblk) {
    if (!st->need_decay) return;
    int pushed = 0;
    for (int q = 0; q < nblk; ++q) pushed += blk[q];
    st->q_size += pushed;
    st->tot = 0;
    st->decays += 1;
}

// ---- inserted mass (sketch.cpp:90): tot += v for every lookup, in double, blocks in order ----------------
__global__ void __launch_bounds__(SG_TPB) k_sg_mass(const float* __restrict__ imp, int n, double* __restrict__ partial) {
    __shared__ double sh[SG_TPB];
    double a = 0.0;
    for (int q = 0; q < SG_BLK / SG_TPB; ++q) {
        const int i = blockIdx.x * SG_BLK + q * SG_TPB + threadIdx.x;
        if (i < n) a += (double)imp[i];
    }
    sh[threadIdx.x] = a;
    __syncthreads();
    for (int o = SG_TPB / 2; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
__global__ void k_sg_mass_end(SgState* st, const double* __restrict__ partial, int nblk, int n, int unit) {
    double a = 0.0;
    if (unit) a = (double)n;
    else for (int q = 0; q < nblk; ++q) a += partial[q];
    st->tot += a;
}

// ---- the two replays ---------------------------------------------------------------------------------------
__global__ void k_sg_keys(const uint32_t* __restrict__ gid, int n, int s, uint32_t* __restrict__ key) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) key[i] = gid[i] % (uint32_t)s;   // :22-24
}
__global__ void k_sg_starts(const uint32_t* __restrict__ skey, int M, int nb, int32_t* __restrict__ start) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > M) return;
    const int lo = (i == 0) ? 0 : (int)skey[i - 1] + 1;
    const int hi = (i == M) ? nb : (int)skey[i];
    for (int k = lo; k <= hi; ++k) start[k] = i;
}
__global__ void k_sg_gather_counts(const float* __restrict__ imp, const int32_t* __restrict__ ord, int n, float* __restrict__ simp) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) simp[i] = imp[ord[i]];
}

// Insert (sketch.cpp:89-123) of one lookup into a bucket held in registers.  COMMIT = false: pass A (a candidate
// is flagged and given a placeholder row); COMMIT = true: pass B (the candidate's fate is known).
template <bool COMMIT>
__device__ __forceinline__ void sg_insert(SgBucket& b, uint32_t x, float v, float kf, int p, uint8_t* __restrict__ cand,
                                          const int32_t* __restrict__ rank, int32_t q_size, uint32_t q_head,
                                          const uint32_t* __restrict__ ring, uint32_t mask, int32_t* __restrict__ out) {
    int found = -1;
#pragma unroll
    for (int i = 3; i >= 0; --i) if (b.cnt[i] != 0.f && b.val[i] == x) found = i;   // first matching slot
    int got = 0;
    if (found >= 0) {
        int pos = found;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (i != found) continue;
            b.cnt[i] += v;
            if (b.cnt[i] >= kf && b.dic[i] == 0) {   // wants a row; gets one iff the FIFO is not empty (:96-103)
                if (!COMMIT) { cand[p] = 1; b.dic[i] = -1; }
                else if (cand[p] && rank[p] < q_size) { b.dic[i] = (int32_t)ring[(q_head + (uint32_t)rank[p]) & mask]; got = 1; }
            }
        }
        // the slot moves up while its count exceeds its predecessor's (:104-109)
#pragma unroll
        for (int j = 3; j >= 1; --j) {
            if (j == pos && b.cnt[j] > b.cnt[j - 1]) {
                const float c = b.cnt[j]; b.cnt[j] = b.cnt[j - 1]; b.cnt[j - 1] = c;
                const uint32_t y = b.val[j]; b.val[j] = b.val[j - 1]; b.val[j - 1] = y;
                const int32_t d = b.dic[j]; b.dic[j] = b.dic[j - 1]; b.dic[j - 1] = d;
                pos = j - 1;
            }
        }
    } else {
        int empty = -1;
#pragma unroll
        for (int i = 3; i >= 0; --i) if (b.cnt[i] == 0.f) empty = i;   // first empty slot (:113-119)
        if (empty >= 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) if (i == empty) { b.cnt[i] = v; b.val[i] = x; }
        } else if (b.dic[3] == 0) {   // Space-Saving: the last slot changes hands, keeping its count (:120-123)
            b.cnt[3] += v;
            b.val[3] = x;
        }
    }
    if (COMMIT) out[p] = got;
}

template <bool COMMIT>
__global__ void __launch_bounds__(SG_TPB) k_sg_pass(SgBucket* __restrict__ tb, int s, int k, const int32_t* __restrict__ start,
                                                    const int32_t* __restrict__ ord, const uint32_t* __restrict__ sgid,
                                                    const float* __restrict__ simp, uint8_t* __restrict__ cand,
                                                    const int32_t* __restrict__ rank, const SgState* __restrict__ st,
                                                    const uint32_t* __restrict__ ring, uint32_t mask, int32_t* __restrict__ out) {
    const int key = blockIdx.x * blockDim.x + threadIdx.x;
    if (key >= s) return;
    const int i0 = start[key], i1 = start[key + 1];
    if (i0 == i1) return;
    SgBucket b = tb[key];
    const float kf = (float)k;
    const int32_t q_size = COMMIT ? st->q_size : 0;
    const uint32_t q_head = COMMIT ? st->q_head : 0u;
    for (int i = i0; i < i1; ++i)
        sg_insert<COMMIT>(b, sgid[i], simp ? simp[i] : 1.0f, kf, ord[i], cand, rank, q_size, q_head, ring, mask, out);
    if (COMMIT) tb[key] = b;
}

// candidates numbered in position order
__global__ void __launch_bounds__(SG_TPB) k_sg_rank_count(const uint8_t* __restrict__ cand, int n, int32_t* __restrict__ blk) {
    __shared__ int s_warp[SG_TPB / 32];
    int c = 0;
    for (int q = 0; q < SG_BLK / SG_TPB; ++q) {
        const int p = blockIdx.x * SG_BLK + threadIdx.x * (SG_BLK / SG_TPB) + q;
        if (p < n) c += cand[p];
    }
    int tot;
    sg_block_exclusive(c, &tot, s_warp);
    if (threadIdx.x == 0) blk[blockIdx.x] = tot;
}
__global__ void __launch_bounds__(SG_TPB) k_sg_rank_write(const uint8_t* __restrict__ cand, int n, const int32_t* __restrict__ blk,
                                                          int32_t* __restrict__ rank, SgState* st) {
    __shared__ int s_warp[SG_TPB / 32];
    const int base = sg_blocks_before(blk, s_warp);
    constexpr int PER = SG_BLK / SG_TPB;
    const int p0 = blockIdx.x * SG_BLK + threadIdx.x * PER;
    int c[PER], cnt = 0;
#pragma unroll
    for (int q = 0; q < PER; ++q) { c[q] = (p0 + q < n) ? cand[p0 + q] : 0; cnt += c[q]; }
    int tot;
    int r = base + sg_block_exclusive(cnt, &tot, s_warp);
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        if (p0 + q >= n) break;
        rank[p0 + q] = r;
        r += c[q];
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) st->n_cand = base + tot;
}
__global__ void k_sg_end(SgState* st) {
    const int pops = st->n_cand < st->q_size ? st->n_cand : st->q_size;   // the first q_size candidates got their rows
    st->q_head += (uint32_t)pops;
    st->q_size -= pops;
    st->num += pops;
}

// ---- update (sketch.cpp:61-75): the FIFO rebuilt from the rows the buckets hold --------------------------
__global__ void k_sg_mark_rows(const SgBucket* __restrict__ tb, int s, int lim, uint8_t* __restrict__ used) {
    int key = blockIdx.x * blockDim.x + threadIdx.x;
    if (key >= s) return;
    const SgBucket b = tb[key];
#pragma unroll
    for (int i = 0; i < 4; ++i) if (b.dic[i] > 0 && b.dic[i] < lim) used[b.dic[i]] = 1;
}
__global__ void __launch_bounds__(SG_TPB) k_sg_free_count(const uint8_t* __restrict__ used, int lim, int32_t* __restrict__ blk) {
    __shared__ int s_warp[SG_TPB / 32];
    int c = 0;
    for (int q = 0; q < SG_BLK / SG_TPB; ++q) {
        const int r = blockIdx.x * SG_BLK + threadIdx.x * (SG_BLK / SG_TPB) + q;
        if (r >= 1 && r < lim) c += used[r] ? 0 : 1;
    }
    int tot;
    sg_block_exclusive(c, &tot, s_warp);
    if (threadIdx.x == 0) blk[blockIdx.x] = tot;
}
__global__ void __launch_bounds__(SG_TPB) k_sg_free_write(const uint8_t* __restrict__ used, int lim, const int32_t* __restrict__ blk,
                                                          uint32_t* __restrict__ ring, SgState* st) {
    __shared__ int s_warp[SG_TPB / 32];
    const int base = sg_blocks_before(blk, s_warp);
    constexpr int PER = SG_BLK / SG_TPB;
    const int r0 = blockIdx.x * SG_BLK + threadIdx.x * PER;
    int c = 0;
#pragma unroll
    for (int q = 0; q < PER; ++q) { const int r = r0 + q; if (r >= 1 && r < lim && !used[r]) ++c; }
    int tot;
    int j = base + sg_block_exclusive(c, &tot, s_warp);
#pragma unroll
    for (int q = 0; q < PER; ++q) { const int r = r0 + q; if (r >= 1 && r < lim && !used[r]) ring[j++] = (uint32_t)r; }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) { st->q_head = 0; st->q_size = base + tot; }
}

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
static int sg_fail(const char* where) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return CAFE_OK;
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: %s", where, cudaGetErrorString(e));
    cafe_internal_set_error(buf);
    return CAFE_ERR_CUDA;
}
static void sg_release(SgHandle* H) {
    void* ptrs[] = {H->b, H->ring, H->st, H->key, H->key_tmp, H->skey, H->sgid, H->pos_tmp, H->ord, H->start, H->rank, H->blk,
                    H->sort_scratch, H->simp, H->cand, H->partial};
    for (void* p : ptrs) if (p) cudaFree(p);
    delete H;
}

extern "C" {

int cafe_sigmod_create(void** out, int lim, int threshold, double decay_rate, int max_lookups) {
    if (!out) return CAFE_ERR_ARG;
    *out = nullptr;
    if (lim < 2 || threshold < 1 || max_lookups < 1 || !(decay_rate > 0.0)) return CAFE_ERR_ARG;
    SgHandle* H = new SgHandle();
    H->lim = lim; H->k = threshold; H->dr = decay_rate; H->cap = max_lookups;
    cudaError_t e = cudaGetDevice(&H->device);
    uint32_t rc = 1;
    while (rc < (uint32_t)lim + 1) rc <<= 1;
    H->ring_mask = rc - 1;
    const size_t M = (size_t)max_lookups;
    const size_t nblk = (size_t)((lim > max_lookups ? lim : max_lookups) / SG_BLK + 2);
    auto A = [&](void** p, size_t n) { if (e == cudaSuccess) e = cudaMalloc(p, n ? n : 1); };
    A((void**)&H->b, sizeof(SgBucket) * (size_t)lim); A((void**)&H->ring, 4 * (size_t)rc); A((void**)&H->st, sizeof(SgState));
    A((void**)&H->key, 4 * M); A((void**)&H->key_tmp, 4 * M); A((void**)&H->skey, 4 * M); A((void**)&H->sgid, 4 * M);
    A((void**)&H->pos_tmp, 4 * M); A((void**)&H->ord, 4 * M); A((void**)&H->start, 4 * ((size_t)lim + 1)); A((void**)&H->rank, 4 * M);
    A((void**)&H->blk, 4 * nblk); A((void**)&H->sort_scratch, 4 * cafe_rs_scratch_elems(max_lookups)); A((void**)&H->simp, 4 * M);
    A((void**)&H->cand, M > (size_t)lim + 1 ? M : (size_t)lim + 1); A((void**)&H->partial, 8 * nblk);
    if (e == cudaSuccess) e = cudaMemset(H->b, 0, sizeof(SgBucket) * (size_t)lim);
    if (e == cudaSuccess) {
        SgState s0;
        memset(&s0, 0, sizeof(s0));
        s0.q_size = lim - 1;   // rows 1 .. lim-1 (sketch.cpp:35-36)
        e = cudaMemcpy(H->st, &s0, sizeof(s0), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) { k_sg_iota<<<sg_blocks(lim - 1), SG_TPB>>>(H->ring, lim - 1, 1u); e = cudaDeviceSynchronize(); }
    if (e != cudaSuccess) { cafe_internal_set_error(cudaGetErrorString(e)); sg_release(H); return CAFE_ERR_CUDA; }
    *out = H;
    return CAFE_OK;
}

int cafe_sigmod_destroy(void* h) {
    if (!h) return CAFE_ERR_ARG;
    cudaDeviceSynchronize();
    sg_release((SgHandle*)h);
    return CAFE_OK;
}

int cafe_sigmod_query(void* h, const uint32_t* gid_dev, int n, int32_t* out_dev, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H || n < 0 || (n > 0 && (!gid_dev || !out_dev))) return CAFE_ERR_ARG;
    if (n == 0) return CAFE_OK;
    k_sg_query<<<sg_blocks(n), SG_TPB, 0, (cudaStream_t)stream>>>(H->b, H->lim, gid_dev, n, out_dev);
    return sg_fail("cafe_sigmod_query");
}

int cafe_sigmod_resolve(void* h, const void* ids_dev, int ids_are_int64, int64_t f_offset, int hash_size, int n,
                        uint32_t* gid_out_dev, int32_t* row_out_dev, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H || n < 0 || hash_size < 1 || (n > 0 && (!ids_dev || !gid_out_dev || !row_out_dev))) return CAFE_ERR_ARG;
    if (n == 0) return CAFE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (ids_are_int64) k_sg_resolve<int64_t><<<sg_blocks(n), SG_TPB, 0, st>>>(H->b, H->lim, (const int64_t*)ids_dev, f_offset, hash_size, n, gid_out_dev, row_out_dev);
    else k_sg_resolve<int32_t><<<sg_blocks(n), SG_TPB, 0, st>>>(H->b, H->lim, (const int32_t*)ids_dev, f_offset, hash_size, n, gid_out_dev, row_out_dev);
    return sg_fail("cafe_sigmod_resolve");
}

int cafe_sigmod_post_rows(void* h, const uint32_t* gid_dev, const int32_t* mask_dev, int n, int32_t* post_row_out_dev, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H || n < 0 || (n > 0 && (!gid_dev || !mask_dev || !post_row_out_dev))) return CAFE_ERR_ARG;
    if (n == 0) return CAFE_OK;
    k_sg_post_rows<<<sg_blocks(n), SG_TPB, 0, (cudaStream_t)stream>>>(H->b, H->lim, gid_dev, mask_dev, n, post_row_out_dev);
    return sg_fail("cafe_sigmod_post_rows");
}

int cafe_sigmod_insert(void* h, const uint32_t* gid_dev, const float* imp_dev, int n, int32_t* mask_out_dev, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H || n < 0) return CAFE_ERR_ARG;
    if (n > H->cap) return CAFE_ERR_CAPACITY;
    if (n > 0 && (!gid_dev || !mask_out_dev)) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int s = H->lim;
    const int nbk = sg_blocks(s, SG_BLK);
    // call boundary: decay when the inserted mass has passed 10 * lim * k (also for an empty call, like the reference)
    k_sg_begin<<<1, 1, 0, st>>>(H->st, s, H->k);
    k_sg_decay_count<<<nbk, SG_TPB, 0, st>>>(H->b, s, H->st, H->dr, H->k, H->blk);
    k_sg_decay_apply<<<nbk, SG_TPB, 0, st>>>(H->b, s, H->st, H->dr, H->k, H->blk, H->ring, H->ring_mask);
    k_sg_decay_end<<<1, 1, 0, st>>>(H->st, H->blk, nbk);
    if (n == 0) return sg_fail("cafe_sigmod_insert");
    const int npb = sg_blocks(n, SG_BLK);
    if (imp_dev) k_sg_mass<<<npb, SG_TPB, 0, st>>>(imp_dev, n, H->partial);
    k_sg_mass_end<<<1, 1, 0, st>>>(H->st, H->partial, npb, n, imp_dev ? 0 : 1);
    // lookups by (bucket, position)
    k_sg_keys<<<sg_blocks(n), SG_TPB, 0, st>>>(gid_dev, n, s, H->key);
    int bits = 1;
    while ((1ll << bits) < s) ++bits;
    CafeKeySource src;
    src.key = H->key; src.gid = nullptr; src.nb = 0;
    cudaError_t e = cafe_radix_sort(src, nullptr, H->key_tmp, H->pos_tmp, H->skey, H->ord, n, bits, H->sort_scratch, gid_dev, H->sgid, st);
    if (e != cudaSuccess) { cafe_internal_set_error(cudaGetErrorString(e)); return CAFE_ERR_CUDA; }
    k_sg_starts<<<sg_blocks((int64_t)n + 1), SG_TPB, 0, st>>>(H->skey, n, s, H->start);
    if (imp_dev) k_sg_gather_counts<<<sg_blocks(n), SG_TPB, 0, st>>>(imp_dev, H->ord, n, H->simp);
    const float* simp = imp_dev ? H->simp : nullptr;
    cudaMemsetAsync(H->cand, 0, (size_t)n, st);
    k_sg_pass<false><<<sg_blocks(s), SG_TPB, 0, st>>>(H->b, s, H->k, H->start, H->ord, H->sgid, simp, H->cand, nullptr, H->st, H->ring,
                                                      H->ring_mask, nullptr);
    k_sg_rank_count<<<npb, SG_TPB, 0, st>>>(H->cand, n, H->blk);
    k_sg_rank_write<<<npb, SG_TPB, 0, st>>>(H->cand, n, H->blk, H->rank, H->st);
    k_sg_pass<true><<<sg_blocks(s), SG_TPB, 0, st>>>(H->b, s, H->k, H->start, H->ord, H->sgid, simp, H->cand, H->rank, H->st, H->ring,
                                                     H->ring_mask, mask_out_dev);
    k_sg_end<<<1, 1, 0, st>>>(H->st);
    return sg_fail("cafe_sigmod_insert");
}

int cafe_sigmod_update(void* h, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int nb = sg_blocks(H->lim, SG_BLK);
    cudaMemsetAsync(H->cand, 0, (size_t)H->lim + 1, st);   // (the candidate flags double as the row marks here)
    k_sg_mark_rows<<<sg_blocks(H->lim), SG_TPB, 0, st>>>(H->b, H->lim, H->lim, H->cand);
    k_sg_free_count<<<nb, SG_TPB, 0, st>>>(H->cand, H->lim, H->blk);
    k_sg_free_write<<<nb, SG_TPB, 0, st>>>(H->cand, H->lim, H->blk, H->ring, H->st);
    return sg_fail("cafe_sigmod_update");
}

// Host arrays: val/cnt/dic [4 * lim], queue [lim]; scalars[0..2] = rows handed out, FIFO length, decays.  Synchronises.
int cafe_sigmod_dump(void* h, uint32_t* val, float* cnt, int32_t* dic, uint32_t* queue, int64_t* scalars, double* tot, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H || !scalars) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaStreamSynchronize(st) != cudaSuccess) return sg_fail("cafe_sigmod_dump");
    SgState s;
    if (cudaMemcpy(&s, H->st, sizeof(s), cudaMemcpyDeviceToHost) != cudaSuccess) return sg_fail("cafe_sigmod_dump");
    scalars[0] = s.num; scalars[1] = s.q_size; scalars[2] = s.decays;
    if (tot) *tot = s.tot;
    if (val && cnt && dic) {
        std::vector<SgBucket> hb((size_t)H->lim);
        if (cudaMemcpy(hb.data(), H->b, sizeof(SgBucket) * (size_t)H->lim, cudaMemcpyDeviceToHost) != cudaSuccess) return sg_fail("cafe_sigmod_dump");
        for (int k = 0; k < H->lim; ++k)
            for (int i = 0; i < 4; ++i) {
                val[k * 4 + i] = hb[k].cnt[i] != 0.f ? hb[k].val[i] : 0u;   // a slot's id means something only with a count
                cnt[k * 4 + i] = hb[k].cnt[i];
                dic[k * 4 + i] = hb[k].dic[i];
            }
    }
    if (queue && s.q_size > 0) {
        std::vector<uint32_t> hr((size_t)H->ring_mask + 1);
        if (cudaMemcpy(hr.data(), H->ring, 4 * hr.size(), cudaMemcpyDeviceToHost) != cudaSuccess) return sg_fail("cafe_sigmod_dump");
        for (int i = 0; i < s.q_size; ++i) queue[i] = hr[(s.q_head + (uint32_t)i) & H->ring_mask];
    }
    return CAFE_OK;
}

// Restores the buckets from a checkpoint (arrays as cafe_sigmod_dump writes them) and rebuilds the FIFO like update().
int cafe_sigmod_load(void* h, const uint32_t* val, const float* cnt, const int32_t* dic, int64_t num, double tot, void* stream) {
    SgHandle* H = (SgHandle*)h;
    if (!H || !val || !cnt || !dic) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<SgBucket> hb((size_t)H->lim);
    for (int k = 0; k < H->lim; ++k)
        for (int i = 0; i < 4; ++i) { hb[k].val[i] = val[k * 4 + i]; hb[k].cnt[i] = cnt[k * 4 + i]; hb[k].dic[i] = dic[k * 4 + i]; }
    if (cudaStreamSynchronize(st) != cudaSuccess) return sg_fail("cafe_sigmod_load");
    if (cudaMemcpy(H->b, hb.data(), sizeof(SgBucket) * (size_t)H->lim, cudaMemcpyHostToDevice) != cudaSuccess) return sg_fail("cafe_sigmod_load");
    SgState s;
    memset(&s, 0, sizeof(s));
    s.num = (int32_t)num; s.tot = tot;
    if (cudaMemcpy(H->st, &s, sizeof(s), cudaMemcpyHostToDevice) != cudaSuccess) return sg_fail("cafe_sigmod_load");
    return cafe_sigmod_update(h, stream);
}

}  // extern "C"
