// sketch_cuda.cu -- CUDA backend of the HotSketch engine (sm_100a) and the sketch part of the C ABI.
//
// Kernels here are thin: one thread per main bucket / LRU bucket / batch position calling the
// functions of sketch_core.cuh.  Radix sorts and prefix scans use CUB device primitives with
// temporary storage that is allocated once per handle, so nothing is allocated on the hot path.
//
// Reference being replaced: the single-threaded C++ HotSketch of tricks/sketch.cpp (batch_query
// :260-265, batch_insert_val :281-296, reset :76-116).
#include <cuda_runtime.h>
#include <stdio.h>

#include <cub/cub.cuh>
#include <algorithm>
#include <string>

#include "../../include/cafe_b200.h"
#include "cafe_internal.h"
#include "radix_sort.cuh"
#include "sketch_engine.h"

#define CAFE_TPB 256

static inline int cafe_blocks(int64_t n, int tpb = CAFE_TPB) { return (int)((n + tpb - 1) / tpb); }

// ---------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------
__global__ void k_fill_iota(uint32_t* p, int n, uint32_t first) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = first + (uint32_t)i;
}

// Several byte fills in one launch (the engine clears a handful of small arrays per job and round).
struct CafeFills {
    unsigned char* p[4];
    size_t n[4];
    int v[4];
    int count;
};
__global__ void k_fills(const CafeFills F) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (int s = 0; s < F.count; ++s) {
        unsigned char* p = F.p[s];
        const size_t n = F.n[s];
        const unsigned b = (unsigned)F.v[s] & 0xffu;
        const unsigned w = b * 0x01010101u;
        size_t head = (16 - ((uintptr_t)p & 15)) & 15;
        if (head > n) head = n;
        const size_t body = (n - head) / 16, tail0 = head + 16 * body;
        for (size_t i = tid; i < body; i += nth) reinterpret_cast<uint4*>(p + head)[i] = make_uint4(w, w, w, w);
        for (size_t i = tid; i < head; i += nth) p[i] = (unsigned char)b;
        for (size_t i = tail0 + tid; i < n; i += nth) p[i] = (unsigned char)b;
    }
}

__global__ void k_query(const CafeMainBucket* __restrict__ mb, int n1, const uint32_t* __restrict__ gid, int n,
                        int32_t* __restrict__ out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t x = gid[i];
    const CafeMainBucket* b = &mb[cafe_hash(x, n1)];
    // val and dic share the bucket's first 32-byte sector
    const uint4 v = *reinterpret_cast<const uint4*>(b->val);
    const int4 d = *reinterpret_cast<const int4*>(b->dic);
    int32_t r = 0;
    if (v.w == x && d.w != 0) r = d.w;
    if (v.z == x && d.z != 0) r = d.z;
    if (v.y == x && d.y != 0) r = d.y;
    if (v.x == x && d.x != 0) r = d.x;
    out[i] = r ? -r : (int32_t)x;
}

__global__ void k_post_query(const CafeMainBucket* __restrict__ mb, int n1, const uint32_t* __restrict__ gid, int n,
                             const int32_t* __restrict__ mask, int32_t* __restrict__ out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int32_t r = 0;
    if (mask[i]) { const uint32_t x = gid[i]; r = cafe_probe_hot(mb[cafe_hash(x, n1)], x); }
    out[i] = r;
}

// start[k] = first sorted index whose key is >= k, for k in [0, nb]
// (also zeroes the two counters of the long-bucket list that k_find_hot, the next launch, fills)
__global__ void k_bucket_starts(const uint32_t* __restrict__ skey, int M, int nb, int32_t* __restrict__ start,
                                int32_t* __restrict__ hot_count) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 2) hot_count[i] = 0;
    if (i > M) return;
    const int lo = (i == 0) ? 0 : (int)skey[i - 1] + 1;
    const int hi = (i == M) ? nb : (int)skey[i];
    for (int k = lo; k <= hi; ++k) start[k] = i;
}

// counts in bucket order, so that the replay kernels stream them beside the sorted positions and ids
__global__ void k_gather_counts(const float* __restrict__ imp, const int32_t* __restrict__ ord1, const int32_t* __restrict__ ord2,
                                int M, float* __restrict__ simp1, float* __restrict__ simp2) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M) return;
    simp1[i] = imp[ord1[i]];
    simp2[i] = imp[ord2[i]];
}

// Buckets with at most CAFE_LONG lookups are replayed by their own thread.  Longer ones (the ids at
// the head of the Zipf law put thousands of lookups into one bucket) are fed by the whole warp:
// 32 lanes load 32 lookups at once, the owning lane applies them in order.  The arithmetic stays
// strictly sequential per bucket; only the loads are shared out.
#define CAFE_LONG 16
#define CAFE_FULL 0xffffffffu
// Very long buckets (the head of the Zipf law) are the serial tail of a pass.  They are listed when
// the lookups are sorted, and the first blocks of the grid take one listed bucket per warp, so that
// the tail starts at once and overlaps with everything else; the other blocks skip listed buckets.
#define CAFE_HOT_LEN 256      // a bucket with more lookups than this is listed in the first region (taken first)
#define CAFE_HOT_CAP 512      // size of that region
// (the second region, behind it, has room for every bucket of the table: with a small sketch and large calls every
// bucket is long)
#define CAFE_LIST_BLOCKS (148 * 4)              // blocks of the launch that works through the list
// Long buckets (more lookups in the sorted stretch than a few times the average) are listed at sort
// time and replayed by a warp each, in a launch of their own that runs beside the thread-per-bucket
// launch for all other buckets: the two kinds of work want different register budgets and occupancy.
// count[0] / count[1] = entries of the two regions; a bucket that finds its region full stays unlisted
// and is handled, correctly but serially, by the thread-per-bucket launch.
struct CafeHot {
    const int32_t* list;
    const int32_t* count;
    const uint8_t* flag;
    int32_t cap2;   // capacity of the second region
};
// (also sets every bucket's flag, listed or not, and its cursor beg[k] = start[k])
__global__ void k_find_hot(const int32_t* __restrict__ start, int nb, int hot_len, int long_len, int cap2, int32_t* list,
                           int32_t* count, uint8_t* flag, int32_t* __restrict__ beg) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= nb) return;
    const int s0 = start[k];
    const int len = start[k + 1] - s0;
    beg[k] = s0;
    uint8_t listed = 0;
    if (len > long_len) {
        bool placed = false;
        if (len > hot_len) {
            const int idx = atomicAdd(&count[0], 1);
            if (idx < CAFE_HOT_CAP) { list[idx] = k; listed = 1; placed = true; }
        }
        if (!placed) {
            const int idx = atomicAdd(&count[1], 1);
            if (idx < cap2) { list[CAFE_HOT_CAP + idx] = k; listed = 1; }
        }
    }
    flag[k] = listed;
}
// next listed bucket for this warp (lane 0 owns it; -1 = none left); the cursor is zeroed with the round result
__device__ __forceinline__ int cafe_next_listed(const CafeHot& H, int32_t* cursor, int nb) {
    const int lane = threadIdx.x & 31;
    const int n_hot = min(H.count[0], CAFE_HOT_CAP), n_long = min(H.count[1], H.cap2);
    int w = 0;
    if (lane == 0) w = atomicAdd(cursor, 1);
    w = __shfl_sync(CAFE_FULL, w, 0);
    if (w >= n_hot + n_long) return -1;
    return lane == 0 ? H.list[w < n_hot ? w : CAFE_HOT_CAP + (w - n_hot)] : nb;
}

// Short buckets, staged.  The lookups of a warp's 32 buckets lie in ascending, disjoint ranges of the
// sorted order.  Instead of every thread chasing its own chain of dependent loads (order entry ->
// position -> id and count) one lookup at a time, the warp loads all entries of a tile in parallel,
// lane e taking entry e, and parks them in shared memory; each thread then replays its own bucket
// from there.  cafe_stage_owner finds, for entry number e of the warp's concatenated ranges, the lane
// whose range holds it: the largest lane whose exclusive prefix is <= e.
__device__ __forceinline__ int cafe_stage_owner(int pref, int e) {
    int L = 0;
#pragma unroll
    for (int b = 16; b > 0; b >>= 1) {
        const int cand = L + b;
        const int pc = __shfl_sync(CAFE_FULL, pref, cand & 31);
        if (pc <= e) L = cand;
    }
    return L;
}
__device__ __forceinline__ int cafe_warp_exclusive(int n, int lane, int* total) {
    int inc = n;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(CAFE_FULL, inc, d);
        if (lane >= d) inc += t;
    }
    *total = __shfl_sync(CAFE_FULL, inc, 31);
    return inc - n;
}
#define CAFE_STAGE_MAIN 128   // entries per tile and warp in the main pass

// PART 0: one listed bucket, owned by lane 0 and fed by the whole warp; PART 1: a thread per bucket.
template <int PART>
__device__ __forceinline__ void cafe_main_body(const CafeJob& J, const CafeHot& H, const int k, float (*s_c)[CAFE_STAGE_MAIN],
                                               int (*s_p)[CAFE_STAGE_MAIN], uint32_t (*s_x)[CAFE_STAGE_MAIN],
                                               uint32_t (*s_kf)[CAFE_STAGE_MAIN], float (*s_d)[CAFE_STAGE_MAIN] = nullptr) {
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    CafeMainReplay R;
    int i = 0, iend = 0;
    bool live = k < J.n1;
    if (PART == 1) {
        // everything the thread needs to start is requested at once: whether its bucket is on the long-bucket
        // list, the range of its lookups and, in a round that replays every bucket, the bucket itself
        CafeMainBucket pre;
        int listed = 0, e1 = 0;
        if (live) {
            listed = H.flag[k]; i = J.beg1[k]; e1 = J.start1[k + 1];
            if (J.all_active) pre = J.main_in[k];
        }
        live = live && !listed;
        if (live) live = R.init(J, k, i, J.all_active ? &pre : nullptr);
        if (live) iend = e1;
    } else if (live) {
        i = J.beg1[k];
        live = R.init(J, k, i);
        if (live) iend = J.start1[k + 1];
    }
    const bool is_long = PART == 0 && live;
    if (PART == 1) {
        const bool is_short = live;
        const int n_k = is_short ? max(iend - i, 0) : 0;
        int T;
        const int pref = cafe_warp_exclusive(n_k, lane, &T);
        bool done = !is_short;
        for (int t0 = 0; t0 < T; t0 += CAFE_STAGE_MAIN) {
            const int tn = min(CAFE_STAGE_MAIN, T - t0);
#pragma unroll
            for (int r = 0; r < CAFE_STAGE_MAIN / 32; ++r) {
                if (r * 32 >= tn) break;   // warp-uniform
                const int e = t0 + r * 32 + lane;
                const int L = cafe_stage_owner(pref, e);
                const int iL = __shfl_sync(CAFE_FULL, i, L), pL = __shfl_sync(CAFE_FULL, pref, L);
                int p = INT32_MAX;
                uint32_t x = 0, kf = CAFE_EV_NONE;
                float c = 1.0f;
                if (e < t0 + tn) {
                    const int idx = iL + (e - pL);   // position, id and count come from the same sorted index
                    p = J.ord1[idx]; x = J.sgid1[idx];
                    if (J.simp1) c = J.simp1[idx];
                    if (!J.first_round && p < J.limit) kf = cafe_old_kind(J, p) | (cafe_old_mflag(J, p) << 8);
                }
                s_p[wib][r * 32 + lane] = p; s_x[wib][r * 32 + lane] = x; s_c[wib][r * 32 + lane] = c; s_kf[wib][r * 32 + lane] = kf;
            }
            __syncwarp();
            const int lo = max(pref, t0), hi = min(pref + n_k, t0 + tn);
            for (int j = lo; j < hi && !done; ++j) {
                const int p = s_p[wib][j - t0];
                if (p >= J.limit) { done = true; break; }   // positions ascend inside a bucket
                const uint32_t kf = s_kf[wib][j - t0];
                R.feed(J, p, s_x[wib][j - t0], s_c[wib][j - t0], kf & 0xffu, kf >> 8);
            }
            __syncwarp();
        }
    }
    unsigned m = PART == 0 ? __ballot_sync(CAFE_FULL, is_long) : 0u;
    while (m) {
        const int o = __ffs(m) - 1;
        m &= m - 1;
        const int s = __shfl_sync(CAFE_FULL, i, o), e = __shfl_sync(CAFE_FULL, iend, o);
        bool stop = false;
        bool hvalid = false, hrow = false;   // warp-uniform copy of the owner's view of the id last dealt with
        uint32_t hx = 0;
        int hslot = 0, hbound = 0;
        // two-deep software pipeline: positions of chunk n+2 and the per-lookup data of chunk n+1 are
        // requested before chunk n is processed, so a long bucket pays one load latency, not one per chunk
        int p_nx = (s + lane < e) ? J.ord1[s + lane] : INT32_MAX;
        int p_n2 = (s + 32 + lane < e) ? J.ord1[s + 32 + lane] : INT32_MAX;
        uint32_t x_nx = 0, ok_nx = CAFE_EV_NONE, of_nx = 0;
        float c_nx = 1.0f;
        if (s + lane < e) { x_nx = J.sgid1[s + lane]; if (J.simp1) c_nx = J.simp1[s + lane]; }
        // (the final pass asks of every miss whether the LRU stage handed it a row: that flag byte rides in bits 8-15)
        if (p_nx < J.limit) { ok_nx = cafe_old_kind(J, p_nx); of_nx = cafe_old_mflag(J, p_nx); if (J.final_pass) of_nx |= (uint32_t)J.lflag[p_nx] << 8; }
        // Number of chunks in a row that went through the calm whole-chunk path.  A calm chunk that ends on a multiple
        // of 256 entries of the bucket looks 512 lookups ahead (one id, one position); if that lookup still belongs
        // to the stretch, the next chunk starts the four-chunk path below.  Shorter stretches stay on the chunk path,
        // which needs no start-up loads.  (Starting points on a fixed grid: a later round that differs in the lookups
        // before the stretch still starts at the same entry and finds what the earlier round remembered.)
        int calm_streak = 0, far_at = -1, far_p = INT32_MAX;
        uint32_t far_x = 0;
        for (int base = s; base < e && !stop; base += 32) {
            if (far_at == base && far_x == hx && far_p < hbound && e - base >= 128) {
                // A long calm stretch (the head ids of a skewed field have thousands of lookups per call)
                // goes four chunks at a time: every lane holds four lookups, the conditions of the calm
                // whole-chunk path are checked for all 128, and the 128 counts are added in order by one
                // chain.  Same two-deep prefetch as the chunk loop, at group granularity.
                float acc = 0.f;
                if (lane == o) {
#pragma unroll
                    for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hslot) acc = R.b.cnt[q];
                }
                acc = __shfl_sync(CAFE_FULL, acc, o);
                int gb = base;
                // A stretch that an earlier round of this job has already added up from the same count gives the
                // same sum again: the bucket remembers its last long stretch (where it began and ended, the count
                // it started from and arrived at) and later rounds and the final pass jump over it.  The lookups'
                // flags were left clean by the round that walked the stretch, and only this bucket writes them.
                const int kb = __shfl_sync(CAFE_FULL, k, o);
                const uint32_t acc_in = __float_as_uint(acc);
                if (J.memo1) {
                    const CafeCalmMemo mm = J.memo1[kb];
                    if (mm.serial == J.serial && mm.i0 == base && mm.acc_in == acc_in && mm.x == hx && mm.slot == hslot &&
                        mm.p_last < hbound && mm.i1 <= e) {
                        acc = __uint_as_float(mm.acc_out);
                        gb = mm.i1;
                    }
                }
                const int g_start = gb;
                // Three sets of registers (A, B, C) take turns as the group being added up, the next one and the one after: positions, ids and counts of a group are requested two groups ahead, what depends on its positions
                // (the event kind and flags the previous round left there) one group ahead, and no freshly requested
                // register is touched before its group comes up for its check, a group and a half later.
                // The chain of 128 additions is the only serial part of a group.  The counts of a group are checked and
                // parked in shared memory one group ahead (two buffers), against a bound taken once (the count at the
                // start: counts only grow, so an addend below it is below every later count too).
                int Ap[4], Bp[4], Cp[4];
                uint32_t Ax[4], Bx[4], Cx[4], Aok[4], Bok[4], Cok[4], Aof[4], Bof[4], Cof[4];
                float Ac[4], Bc[4], Cc[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int i0 = gb + 32 * q + lane, i1 = i0 + 128;
                    Ap[q] = i0 < e ? J.ord1[i0] : INT32_MAX;
                    Bp[q] = i1 < e ? J.ord1[i1] : INT32_MAX;
                    Ax[q] = 0; Ac[q] = 1.0f; Bx[q] = 0; Bc[q] = 1.0f;
                    if (i0 < e) { Ax[q] = J.sgid1[i0]; if (J.simp1) Ac[q] = J.simp1[i0]; }
                    if (i1 < e) { Bx[q] = J.sgid1[i1]; if (J.simp1) Bc[q] = J.simp1[i1]; }
                    Cp[q] = INT32_MAX; Cx[q] = 0; Cc[q] = 1.0f; Cok[q] = CAFE_EV_NONE; Cof[q] = 0; Bok[q] = CAFE_EV_NONE; Bof[q] = 0;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    Aok[q] = CAFE_EV_NONE; Aof[q] = 0;
                    if (Ap[q] < J.limit) { Aok[q] = cafe_old_kind(J, Ap[q]); Aof[q] = cafe_old_mflag(J, Ap[q]); }
                }
                const float acc_bound = acc;
                float* const buf0 = s_c[wib];
                float* const buf1 = s_d[wib];
                bool good;
                {
                    bool g = true;
#pragma unroll
                    for (int q = 0; q < 4; ++q) g = g && Ap[q] < hbound && Ax[q] == hx && Ac[q] >= 0.f && Ac[q] <= acc_bound;
                    good = __all_sync(CAFE_FULL, g);
                }
                if (good) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) buf0[32 * q + lane] = Ac[q];
                }
                // what goes back to the chunk pipeline: the first chunk of the first group that is not added up here
                int h_p0 = Ap[0], h_p1 = Ap[1];
                uint32_t h_x = Ax[0], h_ok = Aok[0], h_of = Aof[0];
                float h_c = Ac[0];
                int bsel = 0;
// one group: C is added up, X is checked and parked, Y is requested
#define CAFE_GROUP_STEP(C, X, Y)                                                                                          \
                {                                                                                                         \
                    _Pragma("unroll") for (int q = 0; q < 4; ++q) {                                                       \
                        const int i2 = gb + 256 + 32 * q + lane;                                                          \
                        Y##p[q] = INT32_MAX; Y##x[q] = 0; Y##c[q] = 1.0f;                                                 \
                        if (i2 < e) { Y##p[q] = J.ord1[i2]; Y##x[q] = J.sgid1[i2]; if (J.simp1) Y##c[q] = J.simp1[i2]; }  \
                        X##ok[q] = CAFE_EV_NONE; X##of[q] = 0;                                                            \
                        if (X##p[q] < J.limit) { X##ok[q] = cafe_old_kind(J, X##p[q]); X##of[q] = cafe_old_mflag(J, X##p[q]); } \
                    }                                                                                                     \
                    __syncwarp();                                                                                         \
                    {                                                                                                     \
                        const float4* cv = reinterpret_cast<const float4*>(bsel ? buf1 : buf0);                           \
                        _Pragma("unroll") for (int q = 0; q < 32; ++q) {                                                  \
                            const float4 t = cv[q];                                                                       \
                            acc = acc + t.x; acc = acc + t.y; acc = acc + t.z; acc = acc + t.w;                           \
                        }                                                                                                 \
                    }                                                                                                     \
                    if (!J.final_pass) {                                                                                  \
                        _Pragma("unroll") for (int q = 0; q < 4; ++q) {                                                   \
                            if (C##of[q] != 0) J.mflag[C##p[q]] = 0;                                                      \
                            if (!J.first_round) {                                                                         \
                                if (C##ok[q] != CAFE_EV_NONE) cafe_withdraw_event(J, C##p[q]);                            \
                                if (C##of[q] & CAFE_F_MISS) { J.mark2[cafe_hash(C##x[q], J.n2)] = 1; J.res->miss_changed = 1; } \
                            }                                                                                             \
                        }                                                                                                 \
                    }                                                                                                     \
                    gb += 128;                                                                                            \
                    bool g = true;                                                                                        \
                    _Pragma("unroll") for (int q = 0; q < 4; ++q)                                                         \
                        g = g && X##p[q] < hbound && X##x[q] == hx && X##c[q] >= 0.f && X##c[q] <= acc_bound;             \
                    good = __all_sync(CAFE_FULL, g);                                                                      \
                    bsel ^= 1;                                                                                            \
                    if (good) {                                                                                           \
                        float* const nb = bsel ? buf1 : buf0;                                                             \
                        _Pragma("unroll") for (int q = 0; q < 4; ++q) nb[32 * q + lane] = X##c[q];                        \
                    } else {                                                                                              \
                        h_p0 = X##p[0]; h_p1 = X##p[1]; h_x = X##x[0]; h_ok = X##ok[0]; h_of = X##of[0]; h_c = X##c[0];   \
                    }                                                                                                     \
                }
// the same in a first round, where no position has flags or an event yet: nothing to read there, nothing to clear
// (entries past the bucket's end are read at the last entry and given a position that fails the check)
#define CAFE_GROUP_STEP_FIRST(C, X, Y)                                                                                    \
                {                                                                                                         \
                    _Pragma("unroll") for (int q = 0; q < 4; ++q) {                                                       \
                        const int i2 = gb + 256 + 32 * q + lane, i2c = min(i2, e - 1);                                    \
                        const int yp = J.ord1[i2c];                                                                       \
                        Y##x[q] = J.sgid1[i2c];                                                                           \
                        Y##c[q] = imp1[i2c];                                                                              \
                        Y##p[q] = i2 < e ? yp : INT32_MAX;                                                                \
                    }                                                                                                     \
                    __syncwarp();                                                                                         \
                    {                                                                                                     \
                        const float4* cv = reinterpret_cast<const float4*>(bsel ? buf1 : buf0);                           \
                        _Pragma("unroll") for (int q = 0; q < 32; ++q) {                                                  \
                            const float4 t = cv[q];                                                                       \
                            acc = acc + t.x; acc = acc + t.y; acc = acc + t.z; acc = acc + t.w;                           \
                        }                                                                                                 \
                    }                                                                                                     \
                    gb += 128;                                                                                            \
                    bool g = true;                                                                                        \
                    _Pragma("unroll") for (int q = 0; q < 4; ++q)                                                         \
                        g = g && X##p[q] < hbound && X##x[q] == hx && X##c[q] >= 0.f && X##c[q] <= acc_bound;             \
                    good = __all_sync(CAFE_FULL, g);                                                                      \
                    bsel ^= 1;                                                                                            \
                    if (good) {                                                                                           \
                        float* const nb = bsel ? buf1 : buf0;                                                             \
                        _Pragma("unroll") for (int q = 0; q < 4; ++q) nb[32 * q + lane] = X##c[q];                        \
                    } else {                                                                                              \
                        h_p0 = X##p[0]; h_p1 = X##p[1]; h_x = X##x[0]; h_c = X##c[0];                                     \
                    }                                                                                                     \
                }
                if (J.first_round && !J.final_pass && J.simp1) {
                    const float* __restrict__ imp1 = J.simp1;
                    while (good) {
                        CAFE_GROUP_STEP_FIRST(A, B, C)
                        if (!good) break;
                        CAFE_GROUP_STEP_FIRST(B, C, A)
                        if (!good) break;
                        CAFE_GROUP_STEP_FIRST(C, A, B)
                    }
                } else {
                    while (good) {
                        CAFE_GROUP_STEP(A, B, C)
                        if (!good) break;
                        CAFE_GROUP_STEP(B, C, A)
                        if (!good) break;
                        CAFE_GROUP_STEP(C, A, B)
                    }
                }
#undef CAFE_GROUP_STEP
#undef CAFE_GROUP_STEP_FIRST
                if (gb != base) {
                    if (J.memo1 && g_start == base && gb - base >= 512 && lane == 0) {   // (walked, not jumped: remember it)
                        CafeCalmMemo mm;
                        mm.serial = J.serial; mm.i0 = base; mm.i1 = gb; mm.p_last = J.ord1[gb - 1];
                        mm.acc_in = acc_in; mm.acc_out = __float_as_uint(acc); mm.x = hx; mm.slot = hslot;
                        J.memo1[kb] = mm;
                    }
                    if (lane == o) {
#pragma unroll
                        for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hslot) R.b.cnt[q] = acc;
                        R.i_cur += gb - base;
                    }
                    base = gb;
                    if (base >= e) break;
                    // hand the loaded lookups back to the chunk pipeline
                    p_nx = h_p0; x_nx = h_x; c_nx = h_c; ok_nx = h_ok; of_nx = h_of;
                    if (J.final_pass && p_nx < J.limit) of_nx |= (uint32_t)J.lflag[p_nx] << 8;
                    p_n2 = h_p1;
                }
            }
            const int streak_in = calm_streak;
            calm_streak = 0;
            const int p = p_nx;
            const uint32_t x = x_nx, ok = ok_nx, of = of_nx;
            const float c = c_nx;
            p_nx = p_n2;
            p_n2 = (base + 64 + lane < e) ? J.ord1[base + 64 + lane] : INT32_MAX;
            x_nx = 0; ok_nx = CAFE_EV_NONE; of_nx = 0; c_nx = 1.0f;
            if (base + 32 + lane < e) { x_nx = J.sgid1[base + 32 + lane]; if (J.simp1) c_nx = J.simp1[base + 32 + lane]; }
            if (p_nx < J.limit) { ok_nx = cafe_old_kind(J, p_nx); of_nx = cafe_old_mflag(J, p_nx); if (J.final_pass) of_nx |= (uint32_t)J.lflag[p_nx] << 8; }
            const int n = min(32, e - base);
            // Whole chunk = 32 more lookups of the id the previous step dealt with, whose slot owns a hot
            // row: add the 32 counts in order, write 32 flags, nothing else can happen.
            if (hvalid && hrow && n == 32 && __all_sync(CAFE_FULL, x == hx && p < hbound)) {
                float cnt0 = 0.f;
                if (lane == o) {
#pragma unroll
                    for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hslot) cnt0 = R.b.cnt[q];
                }
                float acc = __shfl_sync(CAFE_FULL, cnt0, o);
                // Far above the threshold (count > 2*thr, every addend in [0, count]) no lookup of the chunk
                // can satisfy the crossing test "cn >= thr && cn - c < thr" (sketch.cpp:218): cn - c stays
                // within two ulps of a value >= 2*thr.  Then all 32 flags are zero and only the sum is
                // needed; otherwise every lane keeps the running count as of its own lookup.
                const bool calm = acc > 2.0f * J.thr && __all_sync(CAFE_FULL, c >= 0.f && c <= acc);
                float my_acc = 0.f;
                // the 32 counts go through shared memory: every lane reads them back as 8 broadcast 16-byte
                // loads and runs the same chain of 32 dependent adds
                s_c[wib][lane] = c;
                __syncwarp();
                {
                    const float4* cv = reinterpret_cast<const float4*>(s_c[wib]);
                    if (calm) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 t = cv[q];
                            acc = acc + t.x; acc = acc + t.y; acc = acc + t.z; acc = acc + t.w;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 t = cv[q];
                            acc = acc + t.x; if (lane == 4 * q) my_acc = acc;
                            acc = acc + t.y; if (lane == 4 * q + 1) my_acc = acc;
                            acc = acc + t.z; if (lane == 4 * q + 2) my_acc = acc;
                            acc = acc + t.w; if (lane == 4 * q + 3) my_acc = acc;
                        }
                    }
                }
                __syncwarp();
                calm_streak = calm ? streak_in + 1 : 0;
                if (calm && calm_streak >= 2 && ((base + 32 - s) & 255) == 0 && base + 32 + 511 < e) {
                    far_at = base + 32; far_x = J.sgid1[far_at + 511]; far_p = J.ord1[far_at + 511];
                }
                if (lane == o) {
#pragma unroll
                    for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hslot) R.b.cnt[q] = acc;
                    R.i_cur += 32;
                }
                if (!J.final_pass) {
                    const bool cr = !calm && (my_acc >= J.thr && my_acc - c < J.thr);   // sketch.cpp:218
                    const uint32_t nf = cr ? CAFE_F_CROSS : 0;
                    if (nf != of) J.mflag[p] = (uint8_t)nf;
                    if (!J.first_round) {
                        if (ok != CAFE_EV_NONE) cafe_withdraw_event(J, p);
                        if (of & CAFE_F_MISS) { J.mark2[cafe_hash(x, J.n2)] = 1; J.res->miss_changed = 1; }
                    }
                }
                continue;
            }
            int j = 0;
            while (j < n) {
                const int pj = __shfl_sync(CAFE_FULL, p, j);
                const uint32_t xj = __shfl_sync(CAFE_FULL, x, j);
                if (pj >= J.limit) { stop = true; break; }
                // Plain run: consecutive lookups of one id that sits in a slot of this bucket, before the
                // next believed event (and, in the final pass, inside the current segment).  While the
                // slot cannot take a free row -- it owns one already, or its count is below the threshold,
                // or the FIFO is believed empty at that position -- a lookup only adds to the count, may
                // cross the threshold and may be a failed pop candidate.  The counts are added in order
                // by a shuffle chain; every lane writes the flags of its own lookup.  The run stops before
                // the first lookup that could take a row; that one goes through the full replay.
                // (several ids of one bucket may alternate: every lane finds the slot of its own id, and the
                // counts of each slot are added in order by that slot's own chain)
                // Lookups of ids that sit in no slot ride along: a main-table miss changes nothing in the bucket
                // (it goes to the LRU stage; whatever it causes comes back as an event at its own position, which
                // bounds the run), so its lane only writes its flags -- unless the lookup carries an own-promotion
                // event or, in the final pass, was handed a row in the LRU stage: those take the full replay.
                uint32_t bv0 = 0, bv1 = 0, bv2 = 0, bv3 = 0;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                int rowmask = 0, bound = 0, tch = 0;
                if (lane == o) {
                    tch = R.touched ? 1 : 0;
                    bv0 = R.b.val[0]; bv1 = R.b.val[1]; bv2 = R.b.val[2]; bv3 = R.b.val[3];
                    a0 = R.b.cnt[0]; a1 = R.b.cnt[1]; a2 = R.b.cnt[2]; a3 = R.b.cnt[3];
                    rowmask = (R.b.dic[0] != 0 ? 1 : 0) | (R.b.dic[1] != 0 ? 2 : 0) | (R.b.dic[2] != 0 ? 4 : 0) | (R.b.dic[3] != 0 ? 8 : 0);
                    bound = min(R.p_ev, J.limit);
                    if (J.final_pass) bound = min(bound, R.seg_end);
                }
                tch = __shfl_sync(CAFE_FULL, tch, o);
                int run = 0;
                bool advanced = false;
                int ms = -1;   // slot of this lane's id (lowest matching slot, as in the replay)
                if (tch) {
                    bv0 = __shfl_sync(CAFE_FULL, bv0, o); bv1 = __shfl_sync(CAFE_FULL, bv1, o);
                    bv2 = __shfl_sync(CAFE_FULL, bv2, o); bv3 = __shfl_sync(CAFE_FULL, bv3, o);
                    rowmask = __shfl_sync(CAFE_FULL, rowmask, o);
                    bound = __shfl_sync(CAFE_FULL, bound, o);
                    ms = (x == bv0) ? 0 : (x == bv1) ? 1 : (x == bv2) ? 2 : (x == bv3) ? 3 : -1;
                    bool pure = lane >= j && lane < n && ms < 0 && p < bound && ok != CAFE_EV_OWN;
                    if (pure && J.final_pass && ((of >> 8) & CAFE_F_GOT) != 0) pure = false;
                    const bool mine = lane >= j && lane < n && p < bound && (ms >= 0 || pure);
                    const unsigned q = __ballot_sync(CAFE_FULL, mine) >> j;
                    run = __ffs(~q) - 1;          // length of the run of set bits starting at lane j
                    if (run < 0) run = 32 - j;    // all remaining lanes qualify
                    if (run > 0) {
                        const int slot_j = __shfl_sync(CAFE_FULL, ms, j);
                        const bool one_id = (__ballot_sync(CAFE_FULL, lane >= j && lane < j + run && x != xj) == 0);
                        hvalid = one_id && slot_j >= 0; hx = xj; hslot = slot_j < 0 ? 0 : slot_j;
                        hrow = slot_j >= 0 && ((rowmask >> slot_j) & 1) != 0; hbound = bound;
                    }
                }
                if (run >= 2) {
                    a0 = __shfl_sync(CAFE_FULL, a0, o); a1 = __shfl_sync(CAFE_FULL, a1, o);
                    a2 = __shfl_sync(CAFE_FULL, a2, o); a3 = __shfl_sync(CAFE_FULL, a3, o);
                    // Every lane adds up the counts of its own slot's lookups from the run's start to itself, in
                    // order, starting from the slot's count: the same additions in the same order as the replay,
                    // without a cross-lane chain.  The 32 counts are read back from shared memory as 8 broadcast
                    // 16-byte loads; `same` has a bit for every lane of the run whose id sits in this lane's slot.
                    float my_acc = (ms == 0) ? a0 : (ms == 1) ? a1 : (ms == 2) ? a2 : a3;
                    const unsigned same = __match_any_sync(CAFE_FULL, ms) & (0xffffffffu << j) & (0xffffffffu >> (31 - lane));
                    s_c[wib][lane] = c;
                    __syncwarp();
                    {
                        const float4* cv = reinterpret_cast<const float4*>(s_c[wib]);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 t = cv[q];
                            if (same & (1u << (4 * q))) my_acc = my_acc + t.x;
                            if (same & (2u << (4 * q))) my_acc = my_acc + t.y;
                            if (same & (4u << (4 * q))) my_acc = my_acc + t.z;
                            if (same & (8u << (4 * q))) my_acc = my_acc + t.w;
                        }
                    }
                    __syncwarp();
                    const bool in_run = lane >= j && lane < j + run;
                    const bool has_row = ms >= 0 && ((rowmask >> ms) & 1) != 0;
                    const bool cd = ms >= 0 && !has_row && my_acc >= J.thr;   // pop candidate (sketch.cpp:221) ...
                    // ... that could succeed: the FIFO is believed non-empty at its op slot (looked up only for candidates)
                    const bool av = in_run && cd && cafe_fifo_nonempty(J, 2 * (int64_t)p);
                    const unsigned blocked = __ballot_sync(CAFE_FULL, av);
                    const int done = blocked ? (__ffs(blocked) - 1 - j) : run;
                    if (done > 0) {
                        const bool in_done = lane >= j && lane < j + done;
                        const unsigned any_cand = __ballot_sync(CAFE_FULL, in_done && cd);
                        // new count of every slot: the running count at its last lookup inside the applied part
                        float e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f;
                        unsigned l0 = __ballot_sync(CAFE_FULL, in_done && ms == 0), l1 = __ballot_sync(CAFE_FULL, in_done && ms == 1);
                        unsigned l2 = __ballot_sync(CAFE_FULL, in_done && ms == 2), l3 = __ballot_sync(CAFE_FULL, in_done && ms == 3);
                        e0 = __shfl_sync(CAFE_FULL, my_acc, l0 ? 31 - __clz(l0) : 0);
                        e1 = __shfl_sync(CAFE_FULL, my_acc, l1 ? 31 - __clz(l1) : 0);
                        e2 = __shfl_sync(CAFE_FULL, my_acc, l2 ? 31 - __clz(l2) : 0);
                        e3 = __shfl_sync(CAFE_FULL, my_acc, l3 ? 31 - __clz(l3) : 0);
                        if (lane == o) {
                            if (l0) R.b.cnt[0] = e0;
                            if (l1) R.b.cnt[1] = e1;
                            if (l2) R.b.cnt[2] = e2;
                            if (l3) R.b.cnt[3] = e3;
                            R.i_cur += done;
                            if (any_cand) R.cand = true;
                        }
                        if (!J.final_pass && in_done && ms >= 0) {
                            const bool cr = (my_acc >= J.thr && my_acc - c < J.thr);   // sketch.cpp:218
                            const uint32_t nf = (cr ? CAFE_F_CROSS : 0) | (cd ? CAFE_F_POP0 : 0);
                            if (nf != of) J.mflag[p] = (uint8_t)nf;
                            if (!J.first_round) {
                                if (ok != CAFE_EV_NONE) cafe_withdraw_event(J, p);
                                if (of & CAFE_F_MISS) { J.mark2[cafe_hash(x, J.n2)] = 1; J.res->miss_changed = 1; }
                            }
                        }
                        if (!J.final_pass && in_done && ms < 0) {   // goes to the LRU stage; that pass writes lflag
                            if (of != CAFE_F_MISS) J.mflag[p] = CAFE_F_MISS;
                            if (!J.first_round && !(of & CAFE_F_MISS)) { J.mark2[cafe_hash(x, J.n2)] = 1; J.res->miss_changed = 1; }   // new visitor
                        }
                        if (done < run) hvalid = false;
                        j += done;
                        advanced = true;
                    }
                }
                if (!advanced) {
                    const float cj = __shfl_sync(CAFE_FULL, c, j);
                    const uint32_t kj = __shfl_sync(CAFE_FULL, ok, j);
                    const uint32_t fj = __shfl_sync(CAFE_FULL, of, j);
                    if (lane == o) R.feed(J, pj, xj, cj, kj, fj);
                    hvalid = false;   // the full replay step may have changed slots, rows or the next event
                    ++j;
                }
            }
        }
    }
    if (live) R.finish(J);
}
template <int PART>
__global__ void __launch_bounds__(128, PART == 1 ? 6 : 1) k_main_pass(const __grid_constant__ CafeJob J, const CafeHot H) {
    __shared__ __align__(16) float s_c[4][CAFE_STAGE_MAIN];  // per warp: counts of the staged tile / of the chunks being added up
    __shared__ int s_p[4][CAFE_STAGE_MAIN];                  // staged positions, ids, old event kind | old flags << 8
    __shared__ uint32_t s_x[4][CAFE_STAGE_MAIN], s_kf[4][CAFE_STAGE_MAIN];
    __shared__ __align__(16) float s_d[PART == 0 ? 4 : 1][CAFE_STAGE_MAIN];   // list launch: the second buffer of the four-chunk path
    if (PART == 1) {
        const int k = blockIdx.x * blockDim.x + threadIdx.x;
        cafe_main_body<1>(J, H, k < J.n1 ? k : J.n1, s_c, s_p, s_x, s_kf);
    } else {
        for (;;) {
            const int k = cafe_next_listed(H, &J.res->list_cursor[J.final_pass ? 2 : 0], J.n1);
            if (k < 0) break;
            cafe_main_body<0>(J, H, k, s_c, s_p, s_x, s_kf, s_d);
        }
    }
}
// Later rounds and the final pass replay only a small share of the buckets.  One warp scans a chunk of consecutive
// buckets for the ones that are wanted (coalesced reads of the per-bucket state), queues them in shared memory
// and then replays them 32 at a time, a bucket per lane: every lane of every replay has work, where the
// thread-per-bucket launch would drag whole warps along for two or three live lanes.
#define CAFE_SCAN_MAIN 256   // buckets scanned per warp
#define CAFE_SCAN_LRU 64
__global__ void __launch_bounds__(128, 6) k_main_pass_sparse(const __grid_constant__ CafeJob J, const CafeHot H, const int its) {
    __shared__ __align__(16) float s_c[4][CAFE_STAGE_MAIN];
    __shared__ int s_p[4][CAFE_STAGE_MAIN];
    __shared__ uint32_t s_x[4][CAFE_STAGE_MAIN], s_kf[4][CAFE_STAGE_MAIN];
    __shared__ int s_q[4][CAFE_SCAN_MAIN];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int lo = (blockIdx.x * 4 + wib) * its * 32;   // a warp scans its * 32 buckets (its <= CAFE_SCAN_MAIN / 32)
    unsigned act = 0;
#pragma unroll
    for (int it = 0; it < CAFE_SCAN_MAIN / 32; ++it) {
        const int k = lo + it * 32 + lane;
        if (it < its && k < J.n1) { bool cond; if (CafeMainReplay::wanted(J, k, &cond) && !H.flag[k]) act |= 1u << it; }
    }
    int nq = 0;
#pragma unroll
    for (int it = 0; it < CAFE_SCAN_MAIN / 32; ++it) {
        const bool a = (act >> it) & 1u;
        const unsigned m = __ballot_sync(CAFE_FULL, a);
        if (a) s_q[wib][nq + __popc(m & ((1u << lane) - 1u))] = lo + it * 32 + lane;
        nq += __popc(m);
    }
    __syncwarp();
    for (int q0 = 0; q0 < nq; q0 += 32) {
        const int k = q0 + lane < nq ? s_q[wib][q0 + lane] : J.n1;
        cafe_main_body<1>(J, H, k, s_c, s_p, s_x, s_kf);
    }
}

// ---- LRU stage, a chunk of misses at a time -----------------------------------------------------------------------
// The lanes [a, n) of a warp hold consecutive main-table misses of one LRU bucket (one lookup per lane, positions
// ascending with the lane); every lane holds the same copy R of the bucket's replay state.
//
// cafe_lru_apply_chunk applies as many leading lookups as have one of the two plain outcomes -- a hit that stays below
// the threshold (count and clock of the slot change, sketch.cpp:236-249 without the promotion) or a miss whose victim
// leaves no trace (no row, count below 5, no free row to ask for: sketch.cpp:252-268) -- all at once, and returns the
// first lane it did not apply.  While only such lookups happen the bucket is a plain LRU stack of depth 4, so what a
// lookup meets does not depend on how the earlier ones were classified, only on which ids were used how recently:
//   1. lane j's lookup is the latest use of its id as seen from lane i if j < i and the id does not occur in between;
//      every lane collects those lanes in a bit mask (the next lane with the same id, from a match over the warp, is
//      passed around through shared memory).  The bucket's own slots follow in order of their clocks, as far as their
//      ids have not been used in the chunk; empty slots count as entries.
//   2. a lookup hits if fewer than four distinct entries were used since the last use of its id (counted in the
//      mask, plus more recent untouched slots if the id was last used before the chunk); otherwise it replaces the
//      fourth most recent entry;
//   3. the count an entry has after a lookup is 1 at the miss that created it (or the slot's count if it was in the
//      bucket already) plus the counts of its later lookups, added in order by the lane itself;
//   4. the run ends before the first hit that reaches the threshold and the first miss whose victim has a row or a
//      count of 5 or more;
//   5. the slot an entry sits in is the slot of the entry it replaced: pointers from lane to lane, resolved by
//      pointer doubling; the entries that are most recent after the last applied lookup are written into their
//      slots, and every applied lane clears the flags and the event of its position.
// Returns `a` when nothing can be applied (the first lookup needs the full replay, or an id is 0 and would match an
// empty slot, or a lookup of count 1 could ask for a free row).  `s_c`: 32 words of this warp in shared memory.
__device__ __forceinline__ int cafe_lru_apply_chunk(const CafeJob& J, CafeLruReplay& R, const int a, const int n, const int lane,
                                                    const int p, const uint32_t x, const float c, const uint32_t kind,
                                                    float* s_c) {
    const bool act = lane >= a && lane < n;
    if (1.0f >= J.thr) return a;
    if (__any_sync(CAFE_FULL, act && x == 0u)) return a;
    // the bucket's slots from most to least recently used; equal clocks: the lower slot is replaced first
    int Ls0 = 0, Ls1 = 0, Ls2 = 0, Ls3 = 0;
    uint32_t Lv0 = 0, Lv1 = 0, Lv2 = 0, Lv3 = 0;
    bool t_ok = true;
#pragma unroll
    for (int s = 0; s < CAFE_SLOTS; ++s) {
        int rk = 0;
#pragma unroll
        for (int u = 0; u < CAFE_SLOTS; ++u)
            if (u != s) rk += (R.b.t[u] > R.b.t[s] || (R.b.t[u] == R.b.t[s] && u > s)) ? 1 : 0;
        if (rk == 0) { Ls0 = s; Lv0 = R.b.val[s]; }
        if (rk == 1) { Ls1 = s; Lv1 = R.b.val[s]; }
        if (rk == 2) { Ls2 = s; Lv2 = R.b.val[s]; }
        if (rk == 3) { Ls3 = s; Lv3 = R.b.val[s]; }
        t_ok = t_ok && R.b.t[s] < 1000000000;
    }
    if (!t_ok) return a;
    const unsigned rangem = ((n >= 32 ? 0u : (1u << n)) - 1u) & ~((1u << a) - 1u);
    const unsigned lt = (1u << lane) - 1u;
    // 1. latest uses before this lane
    const unsigned same = __match_any_sync(CAFE_FULL, x) & rangem;   // lanes of the chunk with this lane's id
    const unsigned prevm = same & lt;
    const int pv = prevm ? 31 - __clz(prevm) : -1;                   // the previous lookup of this id
    const unsigned nextm = same & ~lt & ~(1u << lane);
    reinterpret_cast<int*>(s_c)[lane] = act ? (nextm ? __ffs(nextm) - 1 : 32) : -1;
    __syncwarp();
    unsigned mask = 0;   // bit j: lane j < this lane holds the latest use of its id before this lane
    {
        const int4* nv = reinterpret_cast<const int4*>(s_c);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int4 t = nv[q];
            if (t.x >= lane) mask |= 1u << (4 * q);
            if (t.y >= lane) mask |= 2u << (4 * q);
            if (t.z >= lane) mask |= 4u << (4 * q);
            if (t.w >= lane) mask |= 8u << (4 * q);
        }
    }
    __syncwarp();
    mask &= lt;
    const int D = __popc(mask);
    // slots of the bucket whose ids have not been used in the chunk before this lane
    const bool U0 = (__ballot_sync(CAFE_FULL, act && x == Lv0) & lt) == 0u, U1 = (__ballot_sync(CAFE_FULL, act && x == Lv1) & lt) == 0u;
    const bool U2 = (__ballot_sync(CAFE_FULL, act && x == Lv2) & lt) == 0u, U3 = (__ballot_sync(CAFE_FULL, act && x == Lv3) & lt) == 0u;
    // 2. hit or miss
    const int ms = (x == R.b.val[0]) ? 0 : (x == R.b.val[1]) ? 1 : (x == R.b.val[2]) ? 2 : (x == R.b.val[3]) ? 3 : -1;
    bool hit = false;
    if (pv >= 0) hit = __popc(mask & ~((2u << pv) - 1u)) <= 3;
    else if (ms >= 0) {
        const int qx = ms == Ls0 ? 0 : ms == Ls1 ? 1 : ms == Ls2 ? 2 : 3;
        const int newer = D + ((qx > 0 && U0) ? 1 : 0) + ((qx > 1 && U1) ? 1 : 0) + ((qx > 2 && U2) ? 1 : 0);
        hit = newer <= 3;
    }
    // the entry a miss replaces: the fourth most recent one
    int vw = 0;   // >= 0: last used by that lane; < 0: slot -1 - vw of the bucket as it was
    if (D >= 4) {
        unsigned t = mask;
        t &= ~(1u << (31 - __clz(t))); t &= ~(1u << (31 - __clz(t))); t &= ~(1u << (31 - __clz(t)));
        vw = 31 - __clz(t);
    } else {
        const int want = 4 - D;   // the want-th untouched slot in clock order
        int seen = 0, vs = 0;
        if (U0) { ++seen; if (seen == want) vs = Ls0; }
        if (U1) { ++seen; if (seen == want) vs = Ls1; }
        if (U2) { ++seen; if (seen == want) vs = Ls2; }
        if (U3) { ++seen; if (seen == want) vs = Ls3; }
        vw = -1 - vs;
    }
    // 3. the entry's count after this lookup
    const unsigned misses = __ballot_sync(CAFE_FULL, act && !hit);
    const unsigned upto = same & (lt | (1u << lane));
    const unsigned sm = upto & misses;
    const int m = sm ? 31 - __clz(sm) : -1;   // the miss that created the entry (this lane itself if it misses)
    const unsigned chain = m >= 0 ? (upto & ~((2u << m) - 1u)) : upto;
    float my_acc = 1.0f;
    int32_t my_dic = 0;
    if (m < 0) {
        my_acc = (ms == 0) ? R.b.cnt[0] : (ms == 1) ? R.b.cnt[1] : (ms == 2) ? R.b.cnt[2] : R.b.cnt[3];
        my_dic = (ms == 0) ? R.b.dic[0] : (ms == 1) ? R.b.dic[1] : (ms == 2) ? R.b.dic[2] : R.b.dic[3];
    }
    s_c[lane] = c;
    __syncwarp();
    {
        const float4* cv = reinterpret_cast<const float4*>(s_c);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 t = cv[q];
            if (chain & (1u << (4 * q))) my_acc = my_acc + t.x;
            if (chain & (2u << (4 * q))) my_acc = my_acc + t.y;
            if (chain & (4u << (4 * q))) my_acc = my_acc + t.z;
            if (chain & (8u << (4 * q))) my_acc = my_acc + t.w;
        }
    }
    __syncwarp();
    // 4. where the run ends
    const float vc_l = __shfl_sync(CAFE_FULL, my_acc, vw >= 0 ? vw : 0);
    const int32_t vd_l = __shfl_sync(CAFE_FULL, my_dic, vw >= 0 ? vw : 0);
    bool plain;
    if (hit) plain = !(my_acc >= J.thr) && (m >= 0 || ms >= 0);
    else {
        const int vs = -1 - vw;
        const float vc = vw >= 0 ? vc_l : (vs == 0 ? R.b.cnt[0] : vs == 1 ? R.b.cnt[1] : vs == 2 ? R.b.cnt[2] : R.b.cnt[3]);
        const int32_t vd = vw >= 0 ? vd_l : (vs == 0 ? R.b.dic[0] : vs == 1 ? R.b.dic[1] : vs == 2 ? R.b.dic[2] : R.b.dic[3]);
        plain = vd == 0 && !(vc >= 5.0f);
    }
    const unsigned bad = __ballot_sync(CAFE_FULL, act && !plain);
    const int f = bad ? __ffs(bad) - 1 : n;
    if (f <= a) return a;
    // 5. the slot of every lane's entry: that of the entry it replaced (a miss) or of the miss that created it (a hit)
    int code = hit ? (m >= 0 ? m : -1 - ms) : vw;   // >= 0: the same slot as that lane's entry; < 0: slot -1 - code
#pragma unroll
    for (int it = 0; it < 5; ++it) {
        const int nx = __shfl_sync(CAFE_FULL, code, code >= 0 ? code : 0);
        if (code >= 0) code = nx;
    }
    const int slot = -1 - code;
    // the entries of the chunk among the four most recent after the last applied lookup: that lookup's own, and the
    // three latest uses of other ids before it (slots of the bucket that are still among the four keep their values)
    const int last = f - 1;
    unsigned others = mask & ~(pv >= 0 ? (1u << pv) : 0u);
    int W1 = -1, W2 = -1, W3 = -1;
    if (others) { W1 = 31 - __clz(others); others &= ~(1u << W1); }
    if (others) { W2 = 31 - __clz(others); others &= ~(1u << W2); }
    if (others) { W3 = 31 - __clz(others); }
    W1 = __shfl_sync(CAFE_FULL, W1, last); W2 = __shfl_sync(CAFE_FULL, W2, last); W3 = __shfl_sync(CAFE_FULL, W3, last);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int W = q == 0 ? last : q == 1 ? W1 : q == 2 ? W2 : W3;
        const int k = W >= 0 ? W : 0;
        const uint32_t ex = __shfl_sync(CAFE_FULL, x, k);
        const float ec = __shfl_sync(CAFE_FULL, my_acc, k);
        const int32_t ed = __shfl_sync(CAFE_FULL, my_dic, k);
        const int ep = __shfl_sync(CAFE_FULL, p, k);
        const int es = __shfl_sync(CAFE_FULL, slot, k);
        if (W >= 0) R.set(es, ex, ec, ed, J.t0 + 1 + ep);
    }
    if (lane >= a && lane < f) {   // no flags, no event
        if (!J.first_round && kind != CAFE_EV_NONE) cafe_withdraw_event(J, p);
        J.lflag[p] = 0;
    }
    return f;
}

// One lookup (lane j's) through the full replay on lane `o`, whose state is then copied to the other lanes.  `ev` /
// `ins` are what the previous round left at the lanes' positions, if the caller has loaded them (HAVE_EV).
template <bool HAVE_EV>
__device__ __forceinline__ void cafe_lru_feed_full(const CafeJob& J, CafeLruReplay& R, const int j, const int o, const int lane,
                                                   const int pj, const uint32_t xj, const float cj, const CafeEvent& ev,
                                                   const int32_t ins) {
    if (HAVE_EV) {
        CafeEvent ej;
        ej.x = __shfl_sync(CAFE_FULL, ev.x, j); ej.cnt = __shfl_sync(CAFE_FULL, ev.cnt, j);
        ej.dic = __shfl_sync(CAFE_FULL, ev.dic, j); ej.kind = __shfl_sync(CAFE_FULL, ev.kind, j);
        const int32_t ij = __shfl_sync(CAFE_FULL, ins, j);
        if (lane == o) R.feed(J, pj, xj, cj, &ej, &ij);
    } else {
        if (lane == o) R.feed(J, pj, xj, cj);
    }
#pragma unroll
    for (int q = 0; q < CAFE_SLOTS; ++q) {
        R.b.val[q] = __shfl_sync(CAFE_FULL, R.b.val[q], o); R.b.cnt[q] = __shfl_sync(CAFE_FULL, R.b.cnt[q], o);
        R.b.dic[q] = __shfl_sync(CAFE_FULL, R.b.dic[q], o); R.b.t[q] = __shfl_sync(CAFE_FULL, R.b.t[q], o);
    }
}

// Replays the misses held by lanes [0, n) into the bucket: chunks of plain lookups at once where that pays (at least
// four lookups left; after an attempt that applied fewer than two, the next `gate.len` lookups go one by one), single
// lookups otherwise -- the two plain outcomes in line on every lane's copy of the state, the rest through the full
// replay.  `kind` is the kind of the event the previous round left at the lane's position (unused in a first
// round); `s_c` is room for 32 counts of this warp in shared memory.
struct CafeRunGate { int skip = 0, len = 0; };
template <bool HAVE_EV>
__device__ __forceinline__ void cafe_lru_feed_lanes(const CafeJob& J, CafeLruReplay& R, const int n, const int o, const int lane,
                                                    const int p, const uint32_t x, const float c, const uint32_t kind,
                                                    const CafeEvent& ev, const int32_t ins, float* s_c, CafeRunGate& gate) {
    int a = 0;
    while (a < n) {
        if (gate.skip > 0) --gate.skip;
        else if (R.touched && n - a >= 4) {
            const int f = cafe_lru_apply_chunk(J, R, a, n, lane, p, x, c, kind, s_c);
            if (f - a >= 2) gate.len = 0;
            else { gate.len = gate.len == 0 ? 1 : (gate.len >= 8 ? 8 : 2 * gate.len); gate.skip = gate.len; }
            if (f > a) {
                a = f;
                if (a >= n) break;
                // the lookup the chunk stopped at needs the full replay
                cafe_lru_feed_full<HAVE_EV>(J, R, a, o, lane, __shfl_sync(CAFE_FULL, p, a), __shfl_sync(CAFE_FULL, x, a),
                                            __shfl_sync(CAFE_FULL, c, a), ev, ins);
                ++a;
                continue;
            }
        }
        const int j = a++;
        const int pj = __shfl_sync(CAFE_FULL, p, j);
        const uint32_t xj = __shfl_sync(CAFE_FULL, x, j);
        const float cj = __shfl_sync(CAFE_FULL, c, j);
        if (!R.touched) { cafe_touch(R.b, J.gflip); R.touched = true; }
        const int32_t tp = J.t0 + 1 + pj;
        int hit = -1, vic = -1, t_min = 1000000000;
#pragma unroll
        for (int q = 0; q < CAFE_SLOTS; ++q) {
            if (hit < 0) {
                if (R.b.val[q] == xj) hit = q;
                else if (t_min > R.b.t[q]) { t_min = R.b.t[q]; vic = q; }
            }
        }
        bool fast = false;
        if (hit >= 0) {
            float cnt0 = 0.f;
#pragma unroll
            for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hit) cnt0 = R.b.cnt[q];
            const float cn = cnt0 + cj;
            if (!(cn >= J.thr)) {
#pragma unroll
                for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hit) { R.b.cnt[q] = cn; R.b.t[q] = tp; }
                fast = true;
            }
        } else if (vic >= 0 && !(1.0f >= J.thr)) {
            float vcnt = 0.f;
            int32_t vdic = 0;
#pragma unroll
            for (int q = 0; q < CAFE_SLOTS; ++q) if (q == vic) { vcnt = R.b.cnt[q]; vdic = R.b.dic[q]; }
            if (vdic == 0 && !(vcnt >= 5.0f)) {
                R.set(vic, xj, 1.0f, 0, tp);
                fast = true;
            }
        }
        if (fast) {
            if (lane == j) {
                if (!J.first_round && kind != CAFE_EV_NONE) cafe_withdraw_event(J, p);
                J.lflag[p] = 0;
            }
            continue;
        }
        cafe_lru_feed_full<HAVE_EV>(J, R, j, o, lane, pj, xj, cj, ev, ins);
    }
}
// per warp of the list launch: the misses of a group of eight chunks, and room for the counts a chunk adds up
struct alignas(16) CafeLruStage { float sum[32]; int p[256]; uint32_t x[256]; float c[256]; uint32_t k[256]; };
template <int PART>
__device__ __forceinline__ void cafe_lru_body(const CafeJob& J, const CafeHot& H, const int k, CafeLruStage* st) {
    const int lane = threadIdx.x & 31;
    CafeLruReplay R;
    int jb = 0, jend = 0;
    bool live = k < J.n2;
    if (PART == 1) {
        // as in the main pass: list flag, range and (when every bucket replays) the bucket are requested together
        CafeLruBucket pre;
        int listed = 0, b1 = 0, e1 = 0;
        if (live) {
            listed = H.flag[k]; b1 = J.beg2[k]; e1 = J.start2[k + 1];
            if (J.all_active) pre = J.lru_in[k];
        }
        live = live && !listed;
        if (live) live = R.init(J, k, J.all_active ? &pre : nullptr);
        if (live) { jb = b1; jend = e1; }
    } else if (live) {
        live = R.init(J, k);
        if (live) { jb = J.beg2[k]; jend = J.start2[k + 1]; }
    }
    const bool is_long = PART == 0 && live;
    if (PART == 1 && live) {
        // Most entries of an LRU bucket are lookups that hit the main table.  Eight entries at a time:
        // their positions, ids and counts (consecutive in the sorted order) are requested together, then the
        // flags of those positions, so a thread waits for two load latencies per eight entries.
        bool done = false;
        for (int j = jb; j < jend && !done; j += 8) {
            int pq[8];
            uint32_t fq[8];
            uint32_t xq[8];
            float cq[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                pq[q] = INT32_MAX; xq[q] = 0; cq[q] = 1.0f;
                if (j + q < jend) { pq[q] = J.ord2[j + q]; xq[q] = J.sgid2[j + q]; if (J.simp2) cq[q] = J.simp2[j + q]; }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) fq[q] = (pq[q] < J.limit) ? (uint32_t)J.mflag[pq[q]] : 0u;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (done) break;
                if (pq[q] >= J.limit) { done = true; break; }   // positions ascend inside a bucket
                if (fq[q] & CAFE_F_MISS) R.feed(J, pq[q], xq[q], cq[q]);
            }
        }
    }
    unsigned m = PART == 0 ? __ballot_sync(CAFE_FULL, is_long) : 0u;
    while (m) {
        const int o = __ffs(m) - 1;
        m &= m - 1;
        const int s = __shfl_sync(CAFE_FULL, jb, o), e = __shfl_sync(CAFE_FULL, jend, o);
        bool stop = false;
        // every lane gets its own copy of the bucket's replay state (reads only); lane o writes the result back
        CafeLruReplay W;
        W.init(J, __shfl_sync(CAFE_FULL, k, o));
        CafeRunGate gate;
        // Three-stage pipeline at a granularity of eight chunks (256 entries, eight per lane): positions
        // are requested three groups ahead, the flags of those positions two groups ahead, ids and counts
        // of the misses among them one group ahead, so that every load has a whole iteration to arrive
        // before the next stage needs it.  Most entries of a long LRU bucket are lookups of a hot id that
        // hit the main table; a group without misses costs eight ballots.
        constexpr int GL = 8;
        int p0[GL], p1[GL], p2[GL], p3[GL];
        uint32_t f0[GL], f1[GL], f2[GL], x0[GL], x1[GL], k0[GL], k1[GL];   // k: kind of the event left at a miss's position
        float c0[GL], c1[GL];
        CafeEvent no_ev;
        no_ev.x = 0; no_ev.cnt = 0.f; no_ev.dic = 0; no_ev.kind = CAFE_EV_NONE;
#pragma unroll
        for (int q = 0; q < GL; ++q) {
            const int i0 = s + 32 * q + lane, i1 = i0 + 32 * GL, i2 = i1 + 32 * GL;
            p0[q] = i0 < e ? J.ord2[i0] : INT32_MAX;
            p1[q] = i1 < e ? J.ord2[i1] : INT32_MAX;
            p2[q] = i2 < e ? J.ord2[i2] : INT32_MAX;
        }
#pragma unroll
        for (int q = 0; q < GL; ++q) {
            f0[q] = p0[q] < J.limit ? (uint32_t)J.mflag[p0[q]] : 0u;
            f1[q] = p1[q] < J.limit ? (uint32_t)J.mflag[p1[q]] : 0u;
        }
#pragma unroll
        for (int q = 0; q < GL; ++q) {
            x0[q] = 0; c0[q] = 1.0f; k0[q] = CAFE_EV_NONE;
            if (f0[q] & CAFE_F_MISS) {
                x0[q] = J.sgid2[s + 32 * q + lane]; if (J.simp2) c0[q] = J.simp2[s + 32 * q + lane];
                if (!J.first_round) k0[q] = J.ev[p0[q]].kind;
            }
        }
        for (int base = s; base < e && !stop; base += 32 * GL) {
#pragma unroll
            for (int q = 0; q < GL; ++q) {
                const int i3 = base + 3 * 32 * GL + 32 * q + lane;
                p3[q] = i3 < e ? J.ord2[i3] : INT32_MAX;
                f2[q] = p2[q] < J.limit ? (uint32_t)J.mflag[p2[q]] : 0u;
                x1[q] = 0; c1[q] = 1.0f; k1[q] = CAFE_EV_NONE;
                if (f1[q] & CAFE_F_MISS) {   // (p1 was read at this index of the sorted order)
                    const int i1 = base + 32 * GL + 32 * q + lane;
                    x1[q] = J.sgid2[i1]; if (J.simp2) c1[q] = J.simp2[i1];
                    if (!J.first_round) k1[q] = J.ev[p1[q]].kind;
                }
            }
            // the group's misses are queued in shared memory, in order, and replayed 32 at a time
            int nq = 0;
#pragma unroll
            for (int q = 0; q < GL; ++q) {
                if (stop) break;   // warp-uniform
                const int idx = base + 32 * q + lane;
                // positions ascend inside a bucket: once one lane sees the limit, later entries are beyond it too
                stop = __any_sync(CAFE_FULL, idx < e && p0[q] >= J.limit);
                const bool missed = (f0[q] & CAFE_F_MISS) != 0;
                const unsigned mm = __ballot_sync(CAFE_FULL, missed);
                if (missed) {
                    const int at = nq + __popc(mm & ((1u << lane) - 1u));
                    st->p[at] = p0[q]; st->x[at] = x0[q]; st->c[at] = c0[q]; st->k[at] = k0[q];
                }
                nq += __popc(mm);
            }
            __syncwarp();
            for (int q0 = 0; q0 < nq; q0 += 32) {
                const int n = min(32, nq - q0);
                int pp = 0;
                uint32_t xx = 0, kk = CAFE_EV_NONE;
                float cc = 1.0f;
                if (lane < n) { pp = st->p[q0 + lane]; xx = st->x[q0 + lane]; cc = st->c[q0 + lane]; kk = st->k[q0 + lane]; }
                cafe_lru_feed_lanes<false>(J, W, n, o, lane, pp, xx, cc, kk, no_ev, 0, st->sum, gate);
            }
            __syncwarp();
#pragma unroll
            for (int q = 0; q < GL; ++q) {
                p0[q] = p1[q]; f0[q] = f1[q]; x0[q] = x1[q]; c0[q] = c1[q]; k0[q] = k1[q];
                p1[q] = p2[q]; f1[q] = f2[q];
                p2[q] = p3[q];
            }
        }
        if (lane == o) W.finish(J);
    }
    if (PART == 1 && live) R.finish(J);
}
template <int PART>
__global__ void __launch_bounds__(128, PART == 1 ? 6 : 1) k_lru_pass(const __grid_constant__ CafeJob J, const CafeHot H) {
    __shared__ CafeLruStage st[PART == 0 ? 4 : 1];   // (list launch only)
    if (PART == 1) {
        const int k = blockIdx.x * blockDim.x + threadIdx.x;
        cafe_lru_body<1>(J, H, k < J.n2 ? k : J.n2, nullptr);
    } else {
        for (;;) {
            const int k = cafe_next_listed(H, &J.res->list_cursor[1], J.n2);
            if (k < 0) break;
            cafe_lru_body<0>(J, H, k, &st[threadIdx.x >> 5]);
        }
    }
}
__global__ void __launch_bounds__(128, 6) k_lru_pass_sparse(const __grid_constant__ CafeJob J, const CafeHot H, const int its) {
    __shared__ int s_q[4][CAFE_SCAN_LRU];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int lo = (blockIdx.x * 4 + wib) * its * 32;
    unsigned act = 0;
#pragma unroll
    for (int it = 0; it < CAFE_SCAN_LRU / 32; ++it) {
        const int k = lo + it * 32 + lane;
        if (it < its && k < J.n2) { bool cond; if (CafeLruReplay::wanted(J, k, &cond) && !H.flag[k]) act |= 1u << it; }
    }
    int nq = 0;
#pragma unroll
    for (int it = 0; it < CAFE_SCAN_LRU / 32; ++it) {
        const bool a = (act >> it) & 1u;
        const unsigned m = __ballot_sync(CAFE_FULL, a);
        if (a) s_q[wib][nq + __popc(m & ((1u << lane) - 1u))] = lo + it * 32 + lane;
        nq += __popc(m);
    }
    __syncwarp();
    for (int q0 = 0; q0 < nq; q0 += 32) {
        const int k = q0 + lane < nq ? s_q[wib][q0 + lane] : J.n2;
        cafe_lru_body<1>(J, H, k, nullptr);
    }
}
__global__ void k_mark_cut(const __grid_constant__ CafeJob J, int from, int to, uint8_t* mark_next1) {
    const int p = from + blockIdx.x * blockDim.x + threadIdx.x;
    if (p < to) cafe_mark_cut_position(J, p, mark_next1);
}
__global__ void k_route(const __grid_constant__ CafeJob J) {
    int p = J.begin + blockIdx.x * blockDim.x + threadIdx.x;
    if (p < J.limit) cafe_route_position(J, p);
}
__global__ void k_finalize_positions(const __grid_constant__ CafeJob J) {
    int p = J.begin + blockIdx.x * blockDim.x + threadIdx.x;
    if (p < J.limit) cafe_finalize_position(J, p);
}
// at commit, per bucket of either table: the LRU clock renumbering and the cursors of the sorted order
__global__ void k_commit_tables(const __grid_constant__ CafeJob J, int32_t* beg1, int32_t* beg2) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < J.n2) {
        cafe_lru_tconvert(J, k);
        beg2[k] = cafe_advance_cursor(J.ord2, beg2[k], J.start2[k + 1], J.limit);
    }
    if (k < J.n1) beg1[k] = cafe_advance_cursor(J.ord1, beg1[k], J.start1[k + 1], J.limit);
}
// ---- FIFO timeline (round step 3), sparse -------------------------------------------------------
// A block of CAFE_TL_THREADS threads handles CAFE_TL_BLOCK consecutive positions (resp. list entries),
// CAFE_TL_PER consecutive ones per thread, so that a scan over threads is a scan in position order.
#define CAFE_TL_THREADS 256
#define CAFE_TL_PER (CAFE_TL_BLOCK / CAFE_TL_THREADS)

// exclusive prefix of v over the block's threads (in thread order) and the block total
__device__ __forceinline__ int cafe_block_exclusive_sum(int v, int* total, int* s_warp) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(CAFE_FULL, inc, d);
        if (lane >= d) inc += t;
    }
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int q = 0; q < CAFE_TL_THREADS / 32; ++q) { const int t = s_warp[q]; if (q < w) before += t; all += t; }
    __syncthreads();
    *total = all;
    return before + inc - v;
}
// the same for the FIFO-size transfer functions (composition is associative but not commutative:
// earlier entries are always the left operand)
__device__ __forceinline__ CafeFn cafe_block_exclusive_fn(const CafeFn& v, CafeFn* total, CafeFn* s_warp) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    CafeFn inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        CafeFn t;
        t.a = __shfl_up_sync(CAFE_FULL, inc.a, d); t.b = __shfl_up_sync(CAFE_FULL, inc.b, d);
        t.np = __shfl_up_sync(CAFE_FULL, inc.np, d); t.pad = 0;
        if (lane >= d) inc = cafe_fn_then(t, inc);
    }
    CafeFn exc;   // composition of the earlier lanes of this warp
    exc.a = __shfl_up_sync(CAFE_FULL, inc.a, 1); exc.b = __shfl_up_sync(CAFE_FULL, inc.b, 1);
    exc.np = __shfl_up_sync(CAFE_FULL, inc.np, 1); exc.pad = 0;
    if (lane == 0) exc = cafe_fn_identity();
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    CafeFn before = cafe_fn_identity(), all = cafe_fn_identity();
#pragma unroll
    for (int q = 0; q < CAFE_TL_THREADS / 32; ++q) {
        const CafeFn t = s_warp[q];
        if (q < w) before = cafe_fn_then(before, t);
        all = cafe_fn_then(all, t);
    }
    __syncthreads();
    *total = all;
    return cafe_fn_then(before, exc);
}

// 3a, first half: ops and main-table misses per block of positions; per-segment threshold crossings and the
// number of LRU visits as block-wide sums, one atomic per block and counter (a block of consecutive
// positions lies in one segment except at boundaries)
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_tl_count(const __grid_constant__ CafeJob J) {
    __shared__ int s_warp[CAFE_TL_THREADS / 32];
    __shared__ int s_cross;
    const int first = J.begin + blockIdx.x * CAFE_TL_BLOCK;
    const int last = min(first + CAFE_TL_BLOCK, J.limit) - 1;
    if (blockIdx.x == 0 && threadIdx.x == 0) J.tl_blk[2 * gridDim.x] = J.tl_head[0];   // the old list's length, for k_tl_emit
    if (threadIdx.x == 0) s_cross = 0;
    __syncthreads();
    const int seg_first = cafe_segment_of(J, first), seg_last = cafe_segment_of(J, last);
    int ops = 0, miss = 0, cross = 0;
#pragma unroll
    for (int i = 0; i < CAFE_TL_PER; ++i) {
        const int p = first + threadIdx.x * CAFE_TL_PER + i;
        if (p >= J.limit) break;
        ops += cafe_ops_count(cafe_ops_of(J, p));
        int c, mi;
        cafe_position_counts(J, p, &c, &mi);
        miss += mi;
        if (c) { if (seg_first == seg_last) ++cross; else atomicAdd(&J.res->seg_real_delta[cafe_segment_of(J, p)], 1); }
    }
    int tot_ops, tot_miss;
    cafe_block_exclusive_sum(ops, &tot_ops, s_warp);
    cafe_block_exclusive_sum(miss, &tot_miss, s_warp);
    if (cross) atomicAdd(&s_cross, cross);
    __syncthreads();
    if (threadIdx.x == 0) {
        J.tl_blk[2 * blockIdx.x] = tot_ops;
        J.tl_blk[2 * blockIdx.x + 1] = tot_miss;
        if (s_cross) atomicAdd(&J.res->seg_real_delta[seg_first], s_cross);
        if (tot_miss) atomicAdd(&J.res->n_miss, tot_miss);
    }
}
// sum of the per-block counts (kind 0: ops, 1: misses) of the blocks ahead of this one
__device__ __forceinline__ int cafe_tl_blocks_before(const CafeJob& J, int kind, int* s_warp) {
    int v = 0;
    for (int q = threadIdx.x; q < (int)blockIdx.x; q += CAFE_TL_THREADS) v += J.tl_blk[2 * q + kind];
    int tot;
    cafe_block_exclusive_sum(v, &tot, s_warp);
    return tot;
}
// 3a, second half: the ops go to their places in the list (updated in place, compared with the old entries)
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_tl_emit(const __grid_constant__ CafeJob J) {
    __shared__ int s_warp[CAFE_TL_THREADS / 32];
    const int first = J.begin + blockIdx.x * CAFE_TL_BLOCK;
    const int32_t n_old = J.tl_blk[2 * gridDim.x];
    const int base = cafe_tl_blocks_before(J, 0, s_warp);
    CafeOps o[CAFE_TL_PER];
    int cnt = 0;
#pragma unroll
    for (int i = 0; i < CAFE_TL_PER; ++i) {
        const int p = first + threadIdx.x * CAFE_TL_PER + i;
        o[i].op0 = o[i].op1 = 0;
        if (p < J.limit) { o[i] = cafe_ops_of(J, p); cnt += cafe_ops_count(o[i]); }
    }
    int tot;
    int j = base + cafe_block_exclusive_sum(cnt, &tot, s_warp);
    const int p0 = first + threadIdx.x * CAFE_TL_PER;
    if (p0 < J.limit && (p0 - J.begin) % CAFE_TL_GROUP == 0) J.tl_grp[(p0 - J.begin) / CAFE_TL_GROUP] = j;
#pragma unroll
    for (int i = 0; i < CAFE_TL_PER; ++i) {
        const int p = p0 + i;
        if (p >= J.limit) break;
        cafe_tl_emit(J, p, o[i], j, n_old);
        j += cafe_ops_count(o[i]);
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        J.tl_grp[(J.limit - J.begin + CAFE_TL_GROUP - 1) / CAFE_TL_GROUP] = base + tot;
        cafe_tl_set_count(J, base + tot, n_old);
    }
}
// 3b, first half: composed transfer function of every block of list entries (the list is usually short: a
// fixed small grid walks over its blocks)
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_tl_aggregate(const __grid_constant__ CafeJob J) {
    __shared__ CafeFn s_warp[CAFE_TL_THREADS / 32];
    const int32_t n = J.tl_head[0];
    for (int blk = blockIdx.x; blk * CAFE_TL_BLOCK < n; blk += gridDim.x) {
        const int base = blk * CAFE_TL_BLOCK;
        CafeFn v = cafe_fn_identity();
#pragma unroll
        for (int i = 0; i < CAFE_TL_PER; ++i) {
            const int j = base + threadIdx.x * CAFE_TL_PER + i;
            if (j < n) v = cafe_fn_then(v, cafe_fn_of_info(J.tl_info[j]));
        }
        CafeFn tot;
        cafe_block_exclusive_fn(v, &tot, s_warp);
        if (threadIdx.x == 0) J.tl_agg[blk] = tot;
    }
}
// 3b, second half: FIFO size and successful pops before every list entry, the pushed rows in order, totals
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_tl_finish(const __grid_constant__ CafeJob J) {
    __shared__ CafeFn s_warp[CAFE_TL_THREADS / 32];
    __shared__ CafeFn s_before;
    const int32_t n = J.tl_head[0];
    for (int blk = blockIdx.x; blk * CAFE_TL_BLOCK < n; blk += gridDim.x) {
        const int base = blk * CAFE_TL_BLOCK;
        if (threadIdx.x == 0) {
            CafeFn f = cafe_fn_identity();
            for (int q = 0; q < blk; ++q) f = cafe_fn_then(f, J.tl_agg[q]);
            s_before = f;
        }
        __syncthreads();
        const int j0 = base + threadIdx.x * CAFE_TL_PER;
        CafeFn v = cafe_fn_identity();
        int32_t info[CAFE_TL_PER];
#pragma unroll
        for (int i = 0; i < CAFE_TL_PER; ++i) {
            info[i] = (j0 + i < n) ? J.tl_info[j0 + i] : 0;
            if (j0 + i < n) v = cafe_fn_then(v, cafe_fn_of_info(info[i]));
        }
        CafeFn tot;
        CafeFn before = cafe_fn_then(s_before, cafe_block_exclusive_fn(v, &tot, s_warp));
#pragma unroll
        for (int i = 0; i < CAFE_TL_PER; ++i) {
            if (j0 + i >= n) break;
            cafe_tl_finish_op(J, j0 + i, n, before);
            before = cafe_fn_then(before, cafe_fn_of_info(info[i]));
        }
        __syncthreads();
    }
}
// at commit: main-table misses up to and including every position of the job (the LRU clock numbering)
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_miss_prefix(const __grid_constant__ CafeJob J) {
    __shared__ int s_warp[CAFE_TL_THREADS / 32];
    const int first = J.begin + blockIdx.x * CAFE_TL_BLOCK;
    const int base = cafe_tl_blocks_before(J, 1, s_warp);
    const int p0 = first + threadIdx.x * CAFE_TL_PER;
    int m[CAFE_TL_PER], cnt = 0;
#pragma unroll
    for (int i = 0; i < CAFE_TL_PER; ++i) {
        m[i] = (p0 + i < J.limit && (J.mflag[p0 + i] & CAFE_F_MISS)) ? 1 : 0;
        cnt += m[i];
    }
    int tot;
    int run = base + cafe_block_exclusive_sum(cnt, &tot, s_warp);
#pragma unroll
    for (int i = 0; i < CAFE_TL_PER; ++i) {
        if (p0 + i >= J.limit) break;
        run += m[i];
        J.nmiss[p0 + i] = run;
    }
}
// ---- LRU pass over compacted miss lists --------------------------------------------------------------
// When a small sketch is fed large calls, an LRU bucket's sorted stretch holds thousands of lookups of which
// most hit the main table (all lookups of a hot id lie in one LRU bucket).  Walking them just to skip them
// then dominates the pass, so the lookups that missed the main table in this round are first compacted, in
// the order of the LRU sort (count per block, then emit at the block's offset, as for the FIFO timeline), and
// each bucket replays its slice of the compacted list, a warp per bucket.
struct CafeMissList {
    int32_t* pre;    // [M + 1] misses among the sorted entries before entry i (pre[M] = all of them)
    int32_t* list;   // [M]     sorted-order indices of the misses
    int32_t* blk;    // [blocks] misses per block of CAFE_TL_BLOCK sorted entries
};
__device__ __forceinline__ int cafe_entry_missed(const CafeJob& J, int i) {
    const int p = J.ord2[i];
    return (p >= J.begin && p < J.limit && (J.mflag[p] & CAFE_F_MISS)) ? 1 : 0;
}
// (a later round in which no lookup entered or left the LRU stage keeps the lists of the round before)
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_lru_miss_count(const __grid_constant__ CafeJob J, const CafeMissList L) {
    __shared__ int s_warp[CAFE_TL_THREADS / 32];
    if (!J.all_active && !J.lists_stale && !J.res->miss_changed) return;
    int c = 0;
#pragma unroll
    for (int q = 0; q < CAFE_TL_PER; ++q) {
        const int i = blockIdx.x * CAFE_TL_BLOCK + threadIdx.x * CAFE_TL_PER + q;
        if (i < J.M) c += cafe_entry_missed(J, i);
    }
    int tot;
    cafe_block_exclusive_sum(c, &tot, s_warp);
    if (threadIdx.x == 0) L.blk[blockIdx.x] = tot;
}
__global__ void __launch_bounds__(CAFE_TL_THREADS) k_lru_miss_emit(const __grid_constant__ CafeJob J, const CafeMissList L) {
    __shared__ int s_warp[CAFE_TL_THREADS / 32];
    if (!J.all_active && !J.lists_stale && !J.res->miss_changed) return;
    int v = 0;
    for (int q = threadIdx.x; q < (int)blockIdx.x; q += CAFE_TL_THREADS) v += L.blk[q];
    int base;
    cafe_block_exclusive_sum(v, &base, s_warp);
    const int i0 = blockIdx.x * CAFE_TL_BLOCK + threadIdx.x * CAFE_TL_PER;
    int m[CAFE_TL_PER], c = 0;
#pragma unroll
    for (int q = 0; q < CAFE_TL_PER; ++q) { m[q] = (i0 + q < J.M) ? cafe_entry_missed(J, i0 + q) : 0; c += m[q]; }
    int tot;
    int j = base + cafe_block_exclusive_sum(c, &tot, s_warp);
#pragma unroll
    for (int q = 0; q < CAFE_TL_PER; ++q) {
        if (i0 + q >= J.M) break;
        L.pre[i0 + q] = j;
        if (m[q]) L.list[j++] = i0 + q;
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) L.pre[J.M] = base + tot;
}
__global__ void __launch_bounds__(128) k_lru_pass_compact(const __grid_constant__ CafeJob J, const CafeMissList L) {
    __shared__ __align__(16) float s_c[4][32];   // per warp: the counts of a run being added up
    const int lane = threadIdx.x & 31;
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    for (int k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); k < J.n2; k += nwarps) {
        CafeLruReplay R;   // the same in every lane
        if (!R.init(J, k)) continue;
        const int jb = L.pre[J.start2[k]], jend = L.pre[J.start2[k + 1]];
        CafeRunGate gate;
        // a chunk of 32 misses -- position, id, count and what the previous round left for the position -- is loaded
        // while the previous chunk is replayed
        int p_nx = 0, i_nx = 0; uint32_t x_nx = 0; float c_nx = 1.0f;
        CafeEvent e_nx; e_nx.x = 0; e_nx.cnt = 0.f; e_nx.dic = 0; e_nx.kind = CAFE_EV_NONE;
        if (jb + lane < jend) {
            const int i = L.list[jb + lane];
            p_nx = J.ord2[i]; x_nx = J.sgid2[i]; if (J.simp2) c_nx = J.simp2[i];
            if (!J.first_round) { e_nx = J.ev[p_nx]; i_nx = J.ins_res[p_nx]; }
        }
        for (int base = jb; base < jend; base += 32) {
            const int p = p_nx, ins = i_nx; const uint32_t x = x_nx; const float c = c_nx; const CafeEvent ev = e_nx;
            c_nx = 1.0f;
            if (base + 32 + lane < jend) {
                const int i = L.list[base + 32 + lane];
                p_nx = J.ord2[i]; x_nx = J.sgid2[i]; if (J.simp2) c_nx = J.simp2[i];
                if (!J.first_round) { e_nx = J.ev[p_nx]; i_nx = J.ins_res[p_nx]; }
            }
            const int n = min(32, jend - base);
            cafe_lru_feed_lanes<true>(J, R, n, 0, lane, p, x, c, ev.kind, ev, ins,
                                      s_c[threadIdx.x >> 5], gate);
        }
        if (lane == 0) R.finish(J);
    }
}
__global__ void k_commit_queue(uint32_t* ring, uint32_t mask, uint32_t q_head, int32_t q_size, int32_t n_pop_ok,
                               const uint32_t* __restrict__ pushbuf, int n_push) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n_push) cafe_commit_push(ring, mask, q_head, q_size, n_pop_ok, pushbuf, j);
}

// The golden path: one thread, lookups strictly in order.
__global__ void k_seq_insert(CafeSeqState* Sd, const uint32_t* __restrict__ gid, const float* __restrict__ imp, int n,
                             int32_t* __restrict__ mask) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    CafeSeqState S = *Sd;
    for (int i = 0; i < n; ++i) mask[i] = cafe_seq_insert(S, gid[i], imp ? imp[i] : 1.0f);
    *Sd = S;
}

__global__ void k_advance_cursors(const int32_t* __restrict__ ord, const int32_t* __restrict__ start, int32_t* beg, int nb,
                                  int limit) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < nb) beg[k] = cafe_advance_cursor(ord, beg[k], start[k + 1], limit);
}

// threshold re-fit, step 1: lazy decay of every bucket and number of candidates per bucket
__global__ void k_reset_count(CafeMainBucket* mb, CafeLruBucket* lb, int n1, int n2, uint32_t gflip, float thr,
                              int32_t* __restrict__ cnt) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < n1) {
        CafeMainBucket b = mb[k];
        const uint32_t f0 = b.flip;
        cnt[k] = cafe_reset_touch_count_main(b, gflip, thr);
        if (f0 != b.flip) mb[k] = b;
    } else if (k < n1 + n2) {
        CafeLruBucket b = lb[k - n1];
        const uint32_t f0 = b.flip;
        cnt[k] = cafe_reset_touch_count_lru(b, gflip, thr);
        if (f0 != b.flip) lb[k - n1] = b;
    } else if (k == n1 + n2) {
        cnt[k] = 0;
    }
}
// step 2 (after an exclusive scan of cnt): candidates in canonical order
__global__ void k_reset_emit(const CafeMainBucket* __restrict__ mb, const CafeLruBucket* __restrict__ lb, int n1, int n2,
                             float thr, const int32_t* __restrict__ off, uint32_t* __restrict__ key,
                             int32_t* __restrict__ val) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n1 + n2) return;
    int o = off[k];
    if (k < n1) {
        const CafeMainBucket b = mb[k];
        for (int i = 0; i < CAFE_SLOTS; ++i)
            if (b.cnt[i] >= thr || b.dic[i] != 0) { key[o] = cafe_float_bits(b.cnt[i]); val[o] = k * CAFE_SLOTS + i; ++o; }
    } else {
        const CafeLruBucket b = lb[k - n1];
        for (int i = 0; i < CAFE_SLOTS; ++i)
            if (b.cnt[i] >= thr || b.dic[i] != 0) { key[o] = cafe_float_bits(b.cnt[i]); val[o] = n1 * CAFE_SLOTS + (k - n1) * CAFE_SLOTS + i; ++o; }
    }
}
// step 3 (after the stable sort by count): sketch.cpp:98-115.  Candidates [0, z] (z = l - lim) give
// their rows back to the FIFO in sorted order; candidates (z, l) without a row then take rows from
// the FIFO front in sorted order while it lasts.  Ranks come from one prefix sum over
// (push flag << 32 | needs-row flag).
__global__ void k_reset_flags(const int32_t* __restrict__ val, int l, int z, CafeMainBucket* mb, CafeLruBucket* lb, int n1,
                              int64_t* __restrict__ flags) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= l) return;
    const int32_t d = *cafe_slot_dic(mb, lb, n1, val[i]);
    flags[i] = (i <= z) ? (d != 0 ? (1ll << 32) : 0ll) : (d == 0 ? 1ll : 0ll);
}
__global__ void k_reset_push(const int32_t* __restrict__ val, int z, CafeMainBucket* mb, CafeLruBucket* lb, int n1,
                             const int64_t* __restrict__ pre, uint32_t* ring, uint32_t mask, uint32_t q_head, int32_t q_size) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > z) return;
    int32_t* d = cafe_slot_dic(mb, lb, n1, val[i]);
    if (*d != 0) {
        ring[(q_head + (uint32_t)(q_size + (int32_t)(pre[i] >> 32))) & mask] = (uint32_t)*d;
        *d = 0;
    }
}
__global__ void k_reset_pop(const uint32_t* __restrict__ key, const int32_t* __restrict__ val, int l, int z,
                            CafeMainBucket* mb, CafeLruBucket* lb, int n1, const int64_t* __restrict__ pre,
                            const uint32_t* __restrict__ ring, uint32_t mask, uint32_t q_head, int32_t q_size,
                            int32_t* __restrict__ out) {
    int i = z + 1 + blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= l) return;
    int32_t* d = cafe_slot_dic(mb, lb, n1, val[i]);
    const int64_t pr = pre[i];
    const int32_t rank = (int32_t)(pr & 0xffffffffll);
    const int32_t avail = q_size + (int32_t)(pr >> 32);   // every push lies before z+1
    const bool needs = (*d == 0);
    if (needs && rank < avail) *d = (int32_t)ring[(q_head + (uint32_t)rank) & mask];
    if (i == l - 1) {
        const int32_t needy = rank + (needs ? 1 : 0);
        out[0] = (int32_t)key[z];
        out[1] = (int32_t)(pr >> 32);
        out[2] = needy < avail ? needy : avail;
    }
}

// ---------------------------------------------------------------------------------------------
// backend
// ---------------------------------------------------------------------------------------------
struct CudaBackend {
    cudaStream_t stream = 0;
    cudaError_t err = cudaSuccess;
    void* cub_tmp = nullptr;
    size_t cub_bytes = 0;
    // lane 0 sorts on `stream`; lanes 1 and 2 on side streams with buffers of their own, forked from
    // and joined to `stream`
    static const int LANES = 3;
    // per lane: scratch of the radix sort, intermediate pairs, sorted keys
    int32_t* sort_scratch[LANES] = {nullptr, nullptr, nullptr};
    uint32_t *key_tmp[LANES] = {nullptr, nullptr, nullptr}, *key_out[LANES] = {nullptr, nullptr, nullptr};
    int32_t* pos_tmp[LANES] = {nullptr, nullptr, nullptr};
    const uint32_t* given_key[LANES] = {nullptr, nullptr, nullptr};   // bucket numbers the caller already has (else hashed here)
    CafeMissList miss = {nullptr, nullptr, nullptr};   // compacted misses of the LRU pass (small sketch, large calls)
    CafeCalmMemo* memo1 = nullptr;   // [n1] last long calm stretch of every main bucket (see the list launch of the main pass)
    cudaStream_t side[LANES] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_fork[LANES] = {nullptr, nullptr, nullptr}, ev_join[LANES] = {nullptr, nullptr, nullptr};
    bool side_pending[LANES] = {false, false, false};
    int64_t* scan64 = nullptr;   // [4*(n1+n2)] prefix sums of the threshold re-fit
    int32_t* hot_list[2] = {nullptr, nullptr};   // listed long buckets of the main / LRU table
    int32_t* hot_count[2] = {nullptr, nullptr};
    uint8_t* hot_flag[2] = {nullptr, nullptr};
    int hot_nb[2] = {0, 0};
    int cap = 0;
    void* pinned = nullptr;   // staging for small device-to-host reads

    ~CudaBackend() {
        if (cub_tmp) cudaFree(cub_tmp);
        if (pass_side) { cudaStreamSynchronize(pass_side); cudaStreamDestroy(pass_side); }
        if (pass_ev_fork) cudaEventDestroy(pass_ev_fork);
        if (pass_ev_join) cudaEventDestroy(pass_ev_join);
        for (int i = 0; i < LANES; ++i) {
            if (side[i]) { cudaStreamSynchronize(side[i]); cudaStreamDestroy(side[i]); }
            if (ev_fork[i]) cudaEventDestroy(ev_fork[i]);
            if (ev_join[i]) cudaEventDestroy(ev_join[i]);
            if (sort_scratch[i]) cudaFree(sort_scratch[i]);
            if (key_tmp[i]) cudaFree(key_tmp[i]);
            if (key_out[i]) cudaFree(key_out[i]);
            if (pos_tmp[i]) cudaFree(pos_tmp[i]);
        }
        if (scan64) cudaFree(scan64);
        if (memo1) cudaFree(memo1);
        if (miss.pre) cudaFree(miss.pre);
        if (miss.list) cudaFree(miss.list);
        if (miss.blk) cudaFree(miss.blk);
        for (int i = 0; i < 2; ++i) { if (hot_list[i]) cudaFree(hot_list[i]); if (hot_count[i]) cudaFree(hot_count[i]); if (hot_flag[i]) cudaFree(hot_flag[i]); }
        if (pinned) cudaFreeHost(pinned);
    }
    void check(cudaError_t e) { if (e != cudaSuccess && err == cudaSuccess) err = e; }
    void check_launch() { check(cudaGetLastError()); }
    bool ok() { return err == cudaSuccess; }

    void* alloc(size_t n) { void* p = nullptr; check(cudaMalloc(&p, n ? n : 1)); return p; }
    void free(void* p) { cudaFree(p); }
    void memset(void* p, int v, size_t n) { if (n) { CAFE_PROF(CAFE_P_MEMSET, stream); check(cudaMemsetAsync(p, v, n, stream)); } }
    // up to four memsets as one launch
    void fills(void* p0, int v0, size_t n0, void* p1 = nullptr, int v1 = 0, size_t n1 = 0, void* p2 = nullptr, int v2 = 0,
               size_t n2 = 0, void* p3 = nullptr, int v3 = 0, size_t n3 = 0) {
        CafeFills F;
        F.count = 0;
        void* ps[4] = {p0, p1, p2, p3};
        const int vs[4] = {v0, v1, v2, v3};
        const size_t ns[4] = {n0, n1, n2, n3};
        size_t most = 0;
        for (int i = 0; i < 4; ++i) {
            if (!ps[i] || !ns[i]) continue;
            F.p[F.count] = (unsigned char*)ps[i]; F.v[F.count] = vs[i]; F.n[F.count] = ns[i];
            ++F.count;
            most = ns[i] > most ? ns[i] : most;
        }
        if (!F.count) return;
        CAFE_PROF(CAFE_P_MEMSET, stream);
        const size_t want = (most / 16 + 255) / 256;
        const int blocks = (int)(want < 1 ? 1 : (want > 1184 ? 1184 : want));   // at most 8 per SM
        k_fills<<<blocks, 256, 0, stream>>>(F);
        check_launch();
    }
    void fill_iota(uint32_t* p, int n, uint32_t first) {
        if (n > 0) { k_fill_iota<<<cafe_blocks(n), CAFE_TPB, 0, stream>>>(p, n, first); check_launch(); }
    }
    void copy(void* d, const void* s, size_t n) { if (n) check(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, stream)); }
    void advance_cursors(const int32_t* ord, const int32_t* start, int32_t* beg, int nb, int limit) {
        CAFE_PROF(CAFE_P_COMMIT, stream);
        k_advance_cursors<<<cafe_blocks(nb), CAFE_TPB, 0, stream>>>(ord, start, beg, nb, limit);
        check_launch();
    }
    void h2d(void* d, const void* s, size_t n) {
        check(cudaMemcpyAsync(d, s, n, cudaMemcpyHostToDevice, stream));
        check(cudaStreamSynchronize(stream));
    }
    void d2h(void* d, const void* s, size_t n) {
        if (pinned && n <= 4096) {
            check(cudaMemcpyAsync(pinned, s, n, cudaMemcpyDeviceToHost, stream));
            check(cudaStreamSynchronize(stream));
            memcpy(d, pinned, n);
        } else {
            check(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToHost, stream));
            check(cudaStreamSynchronize(stream));
        }
    }

    bool prepare(int cap_, int n1, int n2) {
        cap = cap_;
        for (int i = 0; i < LANES; ++i) {
            check(cudaMalloc(&key_tmp[i], 4 * (size_t)cap));
            check(cudaMalloc(&key_out[i], 4 * (size_t)cap));
            check(cudaMalloc(&pos_tmp[i], 4 * (size_t)cap));
            check(cudaMalloc(&sort_scratch[i], 4 * cafe_rs_scratch_elems(cap)));
            if (i == 0) continue;
            // (highest priority: the sorts are chains of small kernels that run beside streaming kernels filling every
            // SM; their blocks must not queue behind those)
            int lo = 0, hi = 0;
            check(cudaDeviceGetStreamPriorityRange(&lo, &hi));
            check(cudaStreamCreateWithPriority(&side[i], cudaStreamNonBlocking, hi));
            check(cudaEventCreateWithFlags(&ev_fork[i], cudaEventDisableTiming));
            check(cudaEventCreateWithFlags(&ev_join[i], cudaEventDisableTiming));
        }
        check(cudaMallocHost(&pinned, 4096));
        hot_nb[0] = n1; hot_nb[1] = n2;
        check(cudaMalloc(&miss.pre, 4 * ((size_t)cap + 1)));
        check(cudaMalloc(&miss.list, 4 * (size_t)cap));
        check(cudaMalloc(&miss.blk, 4 * ((size_t)cap / CAFE_TL_BLOCK + 2)));
        check(cudaMalloc(&memo1, sizeof(CafeCalmMemo) * (size_t)n1));
        check(cudaMemsetAsync(memo1, 0, sizeof(CafeCalmMemo) * (size_t)n1, stream));
        for (int i = 0; i < 2; ++i) {
            check(cudaMalloc(&hot_list[i], 4 * ((size_t)CAFE_HOT_CAP + (size_t)hot_nb[i])));
            check(cudaMalloc(&hot_count[i], 8));
            check(cudaMalloc(&hot_flag[i], (size_t)hot_nb[i]));
            check(cudaMemsetAsync(hot_count[i], 0, 8, stream));
            check(cudaMemsetAsync(hot_flag[i], 0, (size_t)hot_nb[i], stream));
        }
        // largest temporary any CUB call below can ask for
        size_t need = 0, b = 0;
        const int ncand = (n1 + n2) * CAFE_SLOTS;
        check(cudaMalloc(&scan64, 8 * (size_t)ncand));
        const int nsort = cap > ncand ? cap : ncand;
        cub::DeviceRadixSort::SortPairs(nullptr, b, (uint32_t*)nullptr, (uint32_t*)nullptr, (int32_t*)nullptr,
                                        (int32_t*)nullptr, nsort, 0, 32, stream);
        need = b > need ? b : need;
        cub::DeviceScan::InclusiveSum(nullptr, b, (int32_t*)nullptr, (int32_t*)nullptr, nsort, stream);
        need = b > need ? b : need;
        cub_bytes = need * 2 + 1024;
        check(cudaMalloc(&cub_tmp, cub_bytes));
        return ok();
    }

    void query(const CafeMainBucket* mb, int n1, const uint32_t* gid, int n, int32_t* out) {
        CAFE_PROF(CAFE_P_QUERY, stream);
        k_query<<<cafe_blocks(n), CAFE_TPB, 0, stream>>>(mb, n1, gid, n, out);
        check_launch();
    }
    void post_query(const CafeMainBucket* mb, int n1, const uint32_t* gid, int n, const int32_t* mask, int32_t* out) {
        CAFE_PROF(CAFE_P_QUERY, stream);
        k_post_query<<<cafe_blocks(n), CAFE_TPB, 0, stream>>>(mb, n1, gid, n, mask, out);
        check_launch();
    }
    static int bits_for(int nb) { int b = 1; while ((1ll << b) < nb) ++b; return b; }

    // positions ordered by (bucket, position): stable LSD radix sort of the bucket index
    void sort_lookups(const uint32_t* gid, int M, int nb, int32_t* ord, uint32_t* sgid, int32_t* start, int32_t* beg, int lane) {
        cudaStream_t st = stream;
        if (lane != 0 && cafe_prof_serialise()) lane = -lane;   // the lane's buffers, the caller's stream
        if (lane > 0) {
            check(cudaEventRecord(ev_fork[lane], stream));
            check(cudaStreamWaitEvent(side[lane], ev_fork[lane], 0));
            st = side[lane];
        }
        const bool aside = lane > 0;
        lane = lane < 0 ? -lane : lane;
        {
        CAFE_PROF(CAFE_P_LOOKUP_SORT, st);
        // the keys are the hashes of the ids (computed in the first pass); the last pass also writes the ids in sorted order
        CafeKeySource src;
        src.key = given_key[lane]; src.gid = gid; src.nb = nb;
        check(cafe_radix_sort(src, nullptr, key_tmp[lane], pos_tmp[lane], key_out[lane], ord, M, bits_for(nb), sort_scratch[lane],
                              gid, sgid, st));
        const int t = (nb == hot_nb[0]) ? 0 : 1;
        k_bucket_starts<<<cafe_blocks((int64_t)M + 1), CAFE_TPB, 0, st>>>(key_out[lane], M, nb, start, hot_count[t]);
        check_launch();
        // A warp feeding one long bucket leaves 31 lanes idle while it loads, so it pays where that bucket would
        // otherwise be a serial tail of the thread-per-bucket launch: more lookups than a few times the average
        // load -- but never more than 64, beyond which one thread's serial replay is the tail whatever the average
        // (a sketch of a few thousand rows fed 65536-id calls has hundreds of lookups in EVERY bucket).
        const int hot_len = std::max(CAFE_HOT_LEN, std::min((int)(16.0 * M / nb), 4096));
        const int long_len = std::max(16, std::min((int)(4.0 * M / nb), 64));
        k_find_hot<<<cafe_blocks(nb), CAFE_TPB, 0, st>>>(start, nb, hot_len, long_len, nb, hot_list[t], hot_count[t], hot_flag[t],
                                                         beg);
        check_launch();
        }
        if (aside) {
            check(cudaEventRecord(ev_join[lane], side[lane]));
            side_pending[lane] = true;
        }
    }
    void gather_counts(const float* imp, const int32_t* ord1, const int32_t* ord2, int M, float* simp1, float* simp2) {
        CAFE_PROF(CAFE_P_LOOKUP_SORT, stream);
        k_gather_counts<<<cafe_blocks(M), CAFE_TPB, 0, stream>>>(imp, ord1, ord2, M, simp1, simp2);
        check_launch();
    }
    // makes `stream` wait for the sorts outstanding on the side lanes (no-op when there are none)
    void sort_join(int which) {
        for (int lane = 1; lane < LANES; ++lane) {
            if (!side_pending[lane] || (which >= 0 && which != lane)) continue;
            check(cudaStreamWaitEvent(stream, ev_join[lane], 0));
            side_pending[lane] = false;
        }
    }
    // the list launch of a pass runs on a high-priority stream beside the thread-per-bucket launch
    cudaStream_t pass_side = nullptr;
    cudaEvent_t pass_ev_fork = nullptr, pass_ev_join = nullptr;
    void pass_fork() {
        if (!pass_side) {
            int lo = 0, hi = 0;
            check(cudaDeviceGetStreamPriorityRange(&lo, &hi));
            check(cudaStreamCreateWithPriority(&pass_side, cudaStreamNonBlocking, hi));
            check(cudaEventCreateWithFlags(&pass_ev_fork, cudaEventDisableTiming));
            check(cudaEventCreateWithFlags(&pass_ev_join, cudaEventDisableTiming));
        }
        check(cudaEventRecord(pass_ev_fork, stream));
        check(cudaStreamWaitEvent(pass_side, pass_ev_fork, 0));
    }
    void pass_join() {
        check(cudaEventRecord(pass_ev_join, pass_side));
        check(cudaStreamWaitEvent(stream, pass_ev_join, 0));
    }
    cudaEvent_t gate_event = nullptr;   // see SketchEngine::set_gate
    void wait_gate() { if (gate_event) check(cudaStreamWaitEvent(stream, gate_event, 0)); }
    CafeHot hot(int t) const { CafeHot h; h.list = hot_list[t]; h.count = hot_count[t]; h.flag = hot_flag[t]; h.cap2 = hot_nb[t]; return h; }
    // buckets a warp of a sparse launch scans, in units of 32: enough warps to fill the GPU first, long scans second
    static int scan_its(int nb, int most) {
        const int its = (int)((nb + 148 * 16 * 32 - 1) / (148 * 16 * 32));
        return its < 1 ? 1 : (its > most ? most : its);
    }
    void main_pass(const CafeJob& J0) {
        CafeJob J = J0;
        J.memo1 = memo1;
        CAFE_PROF_DYN(J.final_pass ? CAFE_P_MAIN_FINAL : (J.all_active ? CAFE_P_MAIN : CAFE_P_MAIN_LATER), stream);
        pass_fork();
        k_main_pass<0><<<CAFE_LIST_BLOCKS, 128, 0, pass_side>>>(J, hot(0));
        check_launch();
        if (J.all_active) k_main_pass<1><<<cafe_blocks(J.n1, 128), 128, 0, stream>>>(J, hot(0));
        else {
            const int its = scan_its(J.n1, CAFE_SCAN_MAIN / 32);
            k_main_pass_sparse<<<cafe_blocks(J.n1, 4 * 32 * its), 128, 0, stream>>>(J, hot(0), its);
        }
        pass_join();
        check_launch();
    }
    void mark_cut(const CafeJob& J, int from, int to, uint8_t* mark_next1) {
        if (to <= from) return;
        CAFE_PROF(CAFE_P_SCAN, stream);
        k_mark_cut<<<cafe_blocks(to - from), CAFE_TPB, 0, stream>>>(J, from, to, mark_next1);
        check_launch();
    }
    void route(const CafeJob& J) {
        CAFE_PROF(CAFE_P_SCAN, stream);
        k_route<<<cafe_blocks(J.limit - J.begin), CAFE_TPB, 0, stream>>>(J);
        check_launch();
    }
    // per-lookup results and the LRU clock numbering, once the rounds have converged
    void finalize(const CafeJob& J) {
        CAFE_PROF(CAFE_P_COMMIT, stream);
        const int cnt = J.limit - J.begin;
        k_miss_prefix<<<cafe_blocks(cnt, CAFE_TL_BLOCK), CAFE_TL_THREADS, 0, stream>>>(J);
        k_finalize_positions<<<cafe_blocks(cnt), CAFE_TPB, 0, stream>>>(J);
        check_launch();
        k_commit_tables<<<cafe_blocks(J.n1 > J.n2 ? J.n1 : J.n2), CAFE_TPB, 0, stream>>>(J, const_cast<int32_t*>(J.beg1),
                                                                                 const_cast<int32_t*>(J.beg2));
        check_launch();
    }
    void lru_pass(const CafeJob& J) {
        CAFE_PROF_DYN(J.all_active ? CAFE_P_LRU : CAFE_P_LRU_LATER, stream);
        if (J.sgid2 && (int64_t)J.M >= 256 * (int64_t)J.n2) {
            // hundreds of sorted entries per LRU bucket, most of them main-table hits: replay compacted miss lists
            const int g = cafe_blocks(J.M, CAFE_TL_BLOCK);
            k_lru_miss_count<<<g, CAFE_TL_THREADS, 0, stream>>>(J, miss);
            k_lru_miss_emit<<<g, CAFE_TL_THREADS, 0, stream>>>(J, miss);
            const int blocks = std::min(cafe_blocks(J.n2, 4), 148 * 8);
            k_lru_pass_compact<<<blocks, 128, 0, stream>>>(J, miss);
            check_launch();
            return;
        }
        pass_fork();
        k_lru_pass<0><<<CAFE_LIST_BLOCKS, 128, 0, pass_side>>>(J, hot(1));
        check_launch();
        if (J.all_active) k_lru_pass<1><<<cafe_blocks(J.n2, 128), 128, 0, stream>>>(J, hot(1));
        else {
            const int its = scan_its(J.n2, CAFE_SCAN_LRU / 32);
            k_lru_pass_sparse<<<cafe_blocks(J.n2, 4 * 32 * its), 128, 0, stream>>>(J, hot(1), its);
        }
        pass_join();
        check_launch();
    }
    void resolve(const CafeJob& J) {
        CAFE_PROF(CAFE_P_RESOLVE, stream);
        const int cnt = J.limit - J.begin;
        const int g = cafe_blocks(cnt, CAFE_TL_BLOCK);
        k_tl_count<<<g, CAFE_TL_THREADS, 0, stream>>>(J);
        k_tl_emit<<<g, CAFE_TL_THREADS, 0, stream>>>(J);
        // the list has at most two entries per position, usually far fewer: a small grid walks over its blocks
        const int go = std::min(cafe_blocks(2 * (int64_t)cnt, CAFE_TL_BLOCK), 148);
        k_tl_aggregate<<<go, CAFE_TL_THREADS, 0, stream>>>(J);
        k_tl_finish<<<go, CAFE_TL_THREADS, 0, stream>>>(J);
        check_launch();
    }
    void commit_queue(uint32_t* ring, uint32_t mask, uint32_t q_head, int32_t q_size, int32_t n_pop_ok,
                      const uint32_t* pushbuf, int n_push) {
        CAFE_PROF(CAFE_P_COMMIT, stream);
        k_commit_queue<<<cafe_blocks(n_push), CAFE_TPB, 0, stream>>>(ring, mask, q_head, q_size, n_pop_ok, pushbuf, n_push);
        check_launch();
    }
    void seq_insert(CafeSeqState* dev, CafeSeqState* S, const uint32_t* gid, const float* imp, int n, int32_t* mask) {
        check(cudaMemcpyAsync(dev, S, sizeof(CafeSeqState), cudaMemcpyHostToDevice, stream));
        CAFE_PROF(CAFE_P_SEQ, stream);
        k_seq_insert<<<1, 32, 0, stream>>>(dev, gid, imp, n, mask);
        check_launch();
        d2h(S, dev, sizeof(CafeSeqState));
    }
    void reset_collect(CafeMainBucket* mb, CafeLruBucket* lb, int n1, int n2, uint32_t gflip, float thr, int32_t* cnt,
                       uint32_t* key, int32_t* val, int32_t* l_out) {
        const int nb = n1 + n2;
        CAFE_PROF(CAFE_P_REFIT, stream);
        k_reset_count<<<cafe_blocks((int64_t)nb + 1), CAFE_TPB, 0, stream>>>(mb, lb, n1, n2, gflip, thr, cnt);
        check_launch();
        size_t b = cub_bytes;
        check(cub::DeviceScan::ExclusiveSum(cub_tmp, b, cnt, cnt, nb + 1, stream));
        k_reset_emit<<<cafe_blocks(nb), CAFE_TPB, 0, stream>>>(mb, lb, n1, n2, thr, cnt, key, val);
        check_launch();
        d2h(l_out, cnt + nb, 4);
    }
    void sort_pairs(const uint32_t* kin, const int32_t* vin, uint32_t* kout, int32_t* vout, int n, int bits) {
        CAFE_PROF(CAFE_P_REFIT, stream);
        size_t b = cub_bytes;
        check(cub::DeviceRadixSort::SortPairs(cub_tmp, b, kin, kout, vin, vout, n, 0, bits, stream));
    }
    void reset_apply(const uint32_t* key, const int32_t* val, int l, int lim, CafeMainBucket* mb, CafeLruBucket* lb,
                     int n1, uint32_t* ring, uint32_t mask, uint32_t q_head, int32_t q_size, int32_t* dev_out,
                     int32_t* out) {
        CAFE_PROF(CAFE_P_REFIT, stream);
        const int z = l - lim;
        k_reset_flags<<<cafe_blocks(l), CAFE_TPB, 0, stream>>>(val, l, z, mb, lb, n1, scan64);
        check_launch();
        size_t b = cub_bytes;
        check(cub::DeviceScan::ExclusiveSum(cub_tmp, b, scan64, scan64, l, stream));
        k_reset_push<<<cafe_blocks((int64_t)z + 1), CAFE_TPB, 0, stream>>>(val, z, mb, lb, n1, scan64, ring, mask, q_head, q_size);
        check_launch();
        k_reset_pop<<<cafe_blocks((int64_t)l - z - 1), CAFE_TPB, 0, stream>>>(key, val, l, z, mb, lb, n1, scan64, ring, mask,
                                                                            q_head, q_size, dev_out);
        check_launch();
        d2h(out, dev_out, 12);
    }
};

// ---------------------------------------------------------------------------------------------
// handle + C ABI (sketch part)
// ---------------------------------------------------------------------------------------------
struct CafeHandle {
    SketchEngine<CudaBackend> eng;
    int device = 0;
    CafeEmbedWorkspace ws;
};

static thread_local std::string g_last_error;
static void set_error(const char* where, cudaError_t e) {
    g_last_error = std::string(where) + ": " + cudaGetErrorString(e);
}

#define CAFE_H(h) CafeHandle* H = (CafeHandle*)(h); if (!H) return CAFE_ERR_ARG

static int finish(CafeHandle* H, int rc, const char* where) {
    if (!H->eng.be.ok()) { set_error(where, H->eng.be.err); return CAFE_ERR_CUDA; }
    return rc;
}

CafeSketchView cafe_internal_view(void* h) {
    CafeHandle* H = (CafeHandle*)h;
    CafeSketchView v;
    v.main = H->eng.main_table(); v.n1 = H->eng.n1; v.n2 = H->eng.n2; v.lim = H->eng.lim; v.cap = H->eng.capacity();
    return v;
}
CafeEmbedWorkspace* cafe_internal_ws(void* h) { return &((CafeHandle*)h)->ws; }
int cafe_internal_insert(void* h, const uint32_t* gid, const float* imp, const int* seg_off, int nseg, int32_t* mask,
                         int32_t* post_row, int mode, cudaStream_t stream) {
    CafeHandle* H = (CafeHandle*)h;
    H->eng.be.stream = stream;
    int rc = H->eng.insert_segments(gid, imp, seg_off, nseg, mask, post_row, mode != CAFE_INSERT_SEQUENTIAL);
    return finish(H, rc, "cafe_sketch_insert");
}
void cafe_internal_presort(void* h, const uint32_t* gid, int n, const uint32_t* key1, const uint32_t* key2, cudaStream_t stream) {
    CafeHandle* H = (CafeHandle*)h;
    H->eng.be.stream = stream;
    H->eng.be.given_key[1] = key1;   // consumed by the two sort_lookups calls of presort
    H->eng.be.given_key[2] = key2;
    H->eng.presort(gid, n);
    H->eng.be.given_key[1] = H->eng.be.given_key[2] = nullptr;
}
void cafe_internal_set_gate(void* h, int seg, cudaEvent_t ev) {
    CafeHandle* H = (CafeHandle*)h;
    H->eng.be.gate_event = ev;
    H->eng.set_gate(ev ? seg : -1);
}
void cafe_internal_set_error(const char* msg) { g_last_error = msg; }

extern "C" {

const char* cafe_last_error(void) { return g_last_error.c_str(); }

int cafe_sketch_create(void** out, int hotn, float threshold, int adjust_thres, double alpha, int max_lookups) {
    if (!out) return CAFE_ERR_ARG;
    *out = nullptr;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("cafe_sketch_create", e); return CAFE_ERR_CUDA; }
    CafeHandle* H = new CafeHandle();
    H->device = dev;
    int rc = H->eng.init(hotn, threshold, adjust_thres, alpha, max_lookups);
    if (rc == CAFE_OK) rc = cafe_embed_ws_init(&H->ws, max_lookups, hotn);
    if (rc != CAFE_OK) {
        if (!H->eng.be.ok()) set_error("cafe_sketch_create", H->eng.be.err);
        delete H;
        return rc;
    }
    cudaError_t se = cudaStreamSynchronize(0);
    if (se != cudaSuccess) { set_error("cafe_sketch_create", se); delete H; return CAFE_ERR_CUDA; }
    *out = H;
    return CAFE_OK;
}

// The per-handle workspace of the embedding entry points (importance, migration, scatter) without a CAFE+ sketch,
// for callers that bring a sketch of another kind (cafe_sigmod_*).  Destroyed with cafe_sketch_destroy.
int cafe_workspace_create(void** out, int hotn, int max_lookups) {
    if (!out) return CAFE_ERR_ARG;
    *out = nullptr;
    if (hotn < 1 || max_lookups < 1) return CAFE_ERR_ARG;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("cafe_workspace_create", e); return CAFE_ERR_CUDA; }
    CafeHandle* H = new CafeHandle();
    H->device = dev;
    int rc = cafe_embed_ws_init(&H->ws, max_lookups, hotn);
    if (rc != CAFE_OK) { delete H; return rc; }
    *out = H;
    return CAFE_OK;
}

int cafe_sketch_destroy(void* h) {
    CAFE_H(h);
    cudaDeviceSynchronize();
    cafe_embed_ws_free(&H->ws);
    delete H;
    return CAFE_OK;
}

int cafe_sketch_query(void* h, const uint32_t* gid_dev, int n, int32_t* out_dev, void* stream) {
    CAFE_H(h);
    if (n < 0 || (n > 0 && (!gid_dev || !out_dev))) return CAFE_ERR_ARG;
    H->eng.be.stream = (cudaStream_t)stream;
    return finish(H, H->eng.query(gid_dev, n, out_dev), "cafe_sketch_query");
}

int cafe_sketch_insert(void* h, const uint32_t* gid_dev, const float* imp_dev, const int* seg_off_host, int nseg,
                       int32_t* mask_dev, int32_t* post_row_dev, int mode, void* stream) {
    CAFE_H(h);
    return cafe_internal_insert(h, gid_dev, imp_dev, seg_off_host, nseg, mask_dev, post_row_dev, mode, (cudaStream_t)stream);
}

int cafe_sketch_refit(void* h, void* stream) {
    CAFE_H(h);
    H->eng.be.stream = (cudaStream_t)stream;
    return finish(H, H->eng.refit_threshold(), "cafe_sketch_refit");
}

int cafe_sketch_sizes(void* h, int* n1, int* n2, int* lim, int* capacity) {
    CAFE_H(h);
    if (n1) *n1 = H->eng.n1;
    if (n2) *n2 = H->eng.n2;
    if (lim) *lim = H->eng.lim;
    if (capacity) *capacity = H->eng.capacity();
    return CAFE_OK;
}

// scalars[0..7] = threshold bits, real_n, num, t, flip bit, FIFO length, calls so far, fused window
int cafe_sketch_scalars(void* h, int64_t* scalars, double* decay_importance) {
    CAFE_H(h);
    if (!scalars) return CAFE_ERR_ARG;
    uint32_t bits;
    memcpy(&bits, &H->eng.thr, 4);
    scalars[0] = bits; scalars[1] = H->eng.real_n; scalars[2] = H->eng.num; scalars[3] = H->eng.t;
    scalars[4] = H->eng.gflip; scalars[5] = H->eng.q_size; scalars[6] = H->eng.batch_num; scalars[7] = H->eng.window;
    if (decay_importance) *decay_importance = H->eng.decay_importance;
    return CAFE_OK;
}

int cafe_sketch_set_scalars(void* h, const int64_t* scalars, double decay_importance) {
    CAFE_H(h);
    if (!scalars) return CAFE_ERR_ARG;
    uint32_t bits = (uint32_t)scalars[0];
    memcpy(&H->eng.thr, &bits, 4);
    H->eng.real_n = (int)scalars[1]; H->eng.num = (int)scalars[2]; H->eng.t = (int)scalars[3];
    H->eng.gflip = (uint32_t)scalars[4]; H->eng.batch_num = (int)scalars[6];
    H->eng.decay_importance = decay_importance;
    return CAFE_OK;
}

int cafe_sketch_tuning(void* h, int window, int round_cap) {
    CAFE_H(h);
    if (window > 0) H->eng.window = window > CAFE_MAX_SEGMENTS ? CAFE_MAX_SEGMENTS : window;
    if (round_cap > 0) H->eng.round_cap = round_cap;
    return CAFE_OK;
}

int cafe_sketch_stats(void* h, int64_t* out13) {
    CAFE_H(h);
    if (!out13) return CAFE_ERR_ARG;
    memcpy(out13, &H->eng.stats, sizeof(CafeSketchStats));
    return CAFE_OK;
}

int cafe_sketch_dump(void* h, uint32_t* mval, float* mcnt, int32_t* mdic, uint8_t* mflip, uint32_t* lval, float* lcnt,
                     int32_t* ldic, int32_t* lt, uint8_t* lflip, uint32_t* queue, void* stream) {
    CAFE_H(h);
    H->eng.be.stream = (cudaStream_t)stream;
    H->eng.dump(mval, mcnt, mdic, mflip, lval, lcnt, ldic, lt, lflip, queue);
    return finish(H, CAFE_OK, "cafe_sketch_dump");
}

int cafe_sketch_load(void* h, const uint32_t* mval, const float* mcnt, const int32_t* mdic, const uint8_t* mflip,
                     const uint32_t* lval, const float* lcnt, const int32_t* ldic, const int32_t* lt, const uint8_t* lflip,
                     const uint32_t* queue, int queue_len, void* stream) {
    CAFE_H(h);
    H->eng.be.stream = (cudaStream_t)stream;
    return finish(H, H->eng.load(mval, mcnt, mdic, mflip, lval, lcnt, ldic, lt, lflip, queue, queue_len), "cafe_sketch_load");
}

}  // extern "C"
