// sketch_core.cuh -- the HotSketch arithmetic, written once for device and host.
//
// Every function here is __host__ __device__: the CUDA kernels call them one bucket (or one batch
// position) per thread, and a CPU build of the same header replays them in plain loops so that the
// parallel algorithm can be checked against the sequential oracle without a GPU.
//
// Algorithm being reproduced: tricks/sketch.cpp of the reference (CAFE+ HotSketch).  The sequential
// semantics are those of insert (:211-231), insertLRU (:161-210), Insert (:232-259), query (:118-128),
// the lazy decay (:130-140) and reset (:76-116).
//
// Parallel insert.  A batch of lookups (positions 0..M-1, possibly several fields' calls laid end
// to end as "segments") is applied in ROUNDS.  A round replays, from the batch-start state,
//   1. every main bucket: its own lookups in position order, merged with the promotion events that
//      the previous round believed would land in it;
//   2. every LRU bucket: the lookups that missed the main table, in position order;
//   3. the free-row FIFO: every candidate pop and every push, in position order.
// Each decision at position p depends only on the batch-start state and on decisions at earlier
// positions, so the prefix of positions whose beliefs are right grows every round; when a round
// consumes exactly the beliefs it produces, all of them are right and its bucket images are the
// state the sequential loop would have left.
#pragma once
#include "cafe_types.h"

#ifndef INT32_MAX
#define INT32_MAX 2147483647
#endif

#if defined(__CUDA_ARCH__)
#define CAFE_ATOMIC_ADD(p, v) atomicAdd((p), (v))
#define CAFE_ATOMIC_EXCH(p, v) atomicExch((p), (v))
#define CAFE_ATOMIC_OR(p, v) atomicOr((p), (v))
#else
static inline int32_t cafe_host_add(int32_t* p, int32_t v) { int32_t o = *p; *p = o + v; return o; }
static inline int32_t cafe_host_exch(int32_t* p, int32_t v) { int32_t o = *p; *p = v; return o; }
static inline int32_t cafe_host_or(int32_t* p, int32_t v) { int32_t o = *p; *p = o | v; return o; }
#define CAFE_ATOMIC_ADD(p, v) cafe_host_add((p), (v))
#define CAFE_ATOMIC_EXCH(p, v) cafe_host_exch((p), (v))
#define CAFE_ATOMIC_OR(p, v) cafe_host_or((p), (v))
#endif

#define CAFE_DECAY_BASE 10000.0   // sketch.cpp:8

// ---- hashing (sketch.cpp:38-43): 64-bit product of the 32-bit id, remainder by the table size ---
CAFE_HD int32_t cafe_hash(uint32_t x, int32_t n) {
    return (int32_t)(((int64_t)x * 1000000007LL) % (int64_t)n);
}

CAFE_HD uint32_t cafe_float_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; __builtin_memcpy(&u, &f, 4); return u;
#endif
}

// ---- lazy decay (sketch.cpp:130-140): float count divided by a double, rounded back to float ----
CAFE_HD void cafe_decay4(float* cnt) {
#pragma unroll
    for (int i = 0; i < CAFE_SLOTS; ++i) cnt[i] = (float)((double)cnt[i] / CAFE_DECAY_BASE);
}
CAFE_HD void cafe_touch(CafeMainBucket& b, uint32_t gflip) {
    if (b.flip != gflip) { b.flip = gflip; cafe_decay4(b.cnt); }
}
CAFE_HD void cafe_touch(CafeLruBucket& b, uint32_t gflip) {
    if (b.flip != gflip) { b.flip = gflip; cafe_decay4(b.cnt); }
}

// ---- query (sketch.cpp:118-128): hot row of x in this bucket, 0 if none --------------------------
CAFE_HD int32_t cafe_probe_hot(const CafeMainBucket& b, uint32_t x) {
#pragma unroll
    for (int i = 0; i < CAFE_SLOTS; ++i)
        if (b.val[i] == x && b.dic[i] != 0) return b.dic[i];
    return 0;
}

// ---- Insert (sketch.cpp:232-259): place a promoted id; returns 1 on success.  On failure
// *pushed = the carried row that goes back to the FIFO (0 if it carried none). --------------------
CAFE_HD int cafe_promote(CafeMainBucket& b, uint32_t x, float count, int32_t carried, int32_t* pushed) {
    // (written with compile-time slot indices throughout so that a bucket held in registers stays there)
    int empty_i = -1, min_i = -1;
    float min_cnt = 1e9f;
    int32_t min_dic = 0;
    *pushed = 0;
#pragma unroll
    for (int i = CAFE_SLOTS - 1; i >= 0; --i) if (b.val[i] == 0) empty_i = i;   // first empty slot
#pragma unroll
    for (int i = 0; i < CAFE_SLOTS; ++i) {
        // the reference scans slots in order and returns at the first empty one: slots after it never
        // take part in the minimum, slots before it do not matter because the empty one wins
        if (b.cnt[i] < min_cnt) { min_cnt = b.cnt[i]; min_i = i; min_dic = b.dic[i]; }
    }
    if (empty_i >= 0) {
#pragma unroll
        for (int i = 0; i < CAFE_SLOTS; ++i) if (i == empty_i) { b.val[i] = x; b.cnt[i] = count; b.dic[i] = carried; }
        return 1;
    }
    if (min_i >= 0 && min_dic == 0) {
#pragma unroll
        for (int i = 0; i < CAFE_SLOTS; ++i) if (i == min_i) { b.cnt[i] += count; b.val[i] = x; b.dic[i] = carried; }
        return 1;
    }
    *pushed = carried;
    return 0;
}

// =================================================================================================
// Sequential form: one thread, lookups in order, state updated in place.  This is the on-device
// golden path (and the fallback when the parallel rounds do not converge within their cap).
// =================================================================================================
struct CafeSeqState {
    CafeMainBucket* mb;
    CafeLruBucket* lb;
    uint32_t* ring;
    uint32_t ring_mask;
    int32_t n1, n2;
    // scalars, updated in place
    float thr;
    uint32_t gflip;
    int32_t real_n, num, t;
    uint32_t q_head;
    int32_t q_size;
    int32_t error;
};

CAFE_HD void cafe_seq_push(CafeSeqState& S, uint32_t id) {
    if (S.q_size > (int32_t)S.ring_mask) { S.error |= 1; return; }
    S.ring[(S.q_head + (uint32_t)S.q_size) & S.ring_mask] = id;
    S.q_size++;
}
CAFE_HD uint32_t cafe_seq_pop(CafeSeqState& S) {
    uint32_t id = S.ring[S.q_head & S.ring_mask];
    S.q_head++;
    S.q_size--;
    return id;
}
CAFE_HD int cafe_seq_promote(CafeSeqState& S, uint32_t x, float count, int32_t carried) {
    CafeMainBucket& b = S.mb[cafe_hash(x, S.n1)];
    cafe_touch(b, S.gflip);
    int32_t pushed;
    int ok = cafe_promote(b, x, count, carried, &pushed);
    if (!ok && pushed != 0) cafe_seq_push(S, (uint32_t)pushed);
    return ok;
}
// insertLRU, sketch.cpp:161-210
CAFE_HD int cafe_seq_insert_lru(CafeSeqState& S, uint32_t x, float count) {
    CafeLruBucket& b = S.lb[cafe_hash(x, S.n2)];
    int p = -1, t_min = 1000000000, got = 0;
    cafe_touch(b, S.gflip);
    for (int i = 0; i < CAFE_SLOTS; ++i) {
        if (b.val[i] == x) {
            b.t[i] = ++S.t;
            b.cnt[i] += count;
            if (b.cnt[i] >= S.thr && b.cnt[i] - count < S.thr) S.real_n++;
            if (b.cnt[i] >= S.thr && S.q_size > 0 && b.dic[i] == 0) {
                b.dic[i] = (int32_t)cafe_seq_pop(S);
                got = 1;
                S.num++;
            }
            if (b.cnt[i] >= S.thr) {
                if (!cafe_seq_promote(S, b.val[i], b.cnt[i], b.dic[i])) got = 0;
                b.val[i] = 0; b.t[i] = 0; b.cnt[i] = 0.0f; b.dic[i] = 0;
            }
            return got;
        }
        if (t_min > b.t[i]) { t_min = b.t[i]; p = i; }
    }
    if (p < 0) { S.error |= 2; return 0; }
    if (b.dic[p] != 0 || b.cnt[p] >= 5.0f) cafe_seq_promote(S, b.val[p], b.cnt[p], b.dic[p]);
    b.val[p] = x;
    b.t[p] = ++S.t;
    b.cnt[p] = 1.0f;
    b.dic[p] = 0;
    if (b.cnt[p] >= S.thr && b.cnt[p] - count < S.thr) S.real_n++;
    if (b.cnt[p] >= S.thr && S.q_size > 0) {
        b.dic[p] = (int32_t)cafe_seq_pop(S);
        got = 1;
        S.num++;
    }
    return got;
}
// insert, sketch.cpp:211-231
CAFE_HD int cafe_seq_insert(CafeSeqState& S, uint32_t x, float count) {
    CafeMainBucket& b = S.mb[cafe_hash(x, S.n1)];
    cafe_touch(b, S.gflip);
    for (int i = 0; i < CAFE_SLOTS; ++i) {
        if (b.val[i] == x) {
            b.cnt[i] += count;
            float c = b.cnt[i];
            int got = 0;
            if (c >= S.thr && c - count < S.thr) S.real_n++;
            if (c >= S.thr && b.dic[i] == 0 && S.q_size > 0) {
                b.dic[i] = (int32_t)cafe_seq_pop(S);
                got = 1;
                S.num++;
            }
            return got;
        }
    }
    return cafe_seq_insert_lru(S, x, count);
}

// =================================================================================================
// Parallel form.
// =================================================================================================
struct alignas(16) CafeFn { int32_t a, b, np, pad; };   // FIFO size transfer s -> max(s + a, b); pushes so far

// The FIFO timeline is kept sparse: one entry per op (a candidate pop or a push), in op-slot order.
#define CAFE_TL_BLOCK 1024    // positions (resp. ops) handled by one block of the timeline kernels
#define CAFE_TL_GROUP 64      // positions per entry of the coarse index into the op list

// per-lookup result flags (one byte written by the main pass, one by the LRU pass)
enum { CAFE_F_MISS = 1, CAFE_F_POP0 = 2, CAFE_F_POP1 = 4, CAFE_F_CROSS = 8, CAFE_F_GOT = 16 };
// per-bucket replay state kept between rounds
enum { CAFE_S_COND = 1, CAFE_S_CAND = 2, CAFE_S_DIRTY = 4 };   // DIRTY: a row was handed out or an event landed

// what a main bucket remembers of its last long stretch of lookups of one hot id (CUDA list launch only)
struct alignas(16) CafeCalmMemo { int32_t serial, i0, i1, p_last; uint32_t acc_in, acc_out, x; int32_t slot; };

struct CafeJob {
    // the lookups
    const uint32_t* gid;     // [M] global ids
    const float* imp;        // [M] counts, or null for unit counts
    int32_t M;               // capacity of the per-lookup arrays (all lookups of the call)
    int32_t begin;           // the job covers positions [begin, limit); earlier ones were committed by earlier jobs
    int32_t limit;
    int32_t nseg;
    int32_t seg_off[CAFE_MAX_SEGMENTS + 1];
    // positions ordered by (main bucket, position) and by (LRU bucket, position); bucket ranges
    const int32_t* ord1;
    const int32_t* start1;   // [n1+1] bucket ranges in ord1 (whole call)
    const int32_t* beg1;     // [n1]   first entry of each bucket that is >= begin
    const int32_t* ord2;
    const int32_t* start2;   // [n2+1]
    const int32_t* beg2;     // [n2]
    // ids and counts permuted into the two orders (sgid1[i] = gid[ord1[i]], ...; simp* null for unit counts): the
    // replay kernels read them beside the positions instead of gathering them by position
    const uint32_t* sgid1;
    const float* simp1;
    const uint32_t* sgid2;
    const float* simp2;
    // batch-start state (read) and the image the rounds write
    const CafeMainBucket* main_in;
    CafeMainBucket* main_out;
    const CafeLruBucket* lru_in;
    CafeLruBucket* lru_out;
    int32_t n1, n2;
    float thr;
    uint32_t gflip;
    int32_t t0;
    // free-row FIFO at batch start
    const uint32_t* ring;
    uint32_t ring_mask;
    uint32_t q_head;
    int32_t q_size;
    int32_t serial;          // number of this job within its sketch (never 0)
    CafeCalmMemo* memo1;     // [n1] or null
    // round control
    int32_t first_round;   // no beliefs exist yet: every bucket replays and nothing old is read
    int32_t all_active;    // every bucket replays (first round, or the job has just been shortened)
    int32_t cand_active;   // the FIFO timeline changed in the previous round: buckets with ids waiting for a row replay
    int32_t lists_stale;   // the job has just been shortened: per-round lists built for the longer window are rebuilt
    int32_t final_pass;    // converged: buckets that handed out or received rows replay once more to
                           // record post_row; nothing else is written
    // beliefs: the promotion event of every position, kept in place and updated by the LRU pass
    CafeEvent* ev;           // [M]
    int32_t* head;           // [n1] newest victim-promotion event per target bucket (-1 = none); rebuilt per round
    int32_t* nxt;            // [M]  next older event with the same target
    uint8_t* mark_own;       // [n1] 1 = one of the bucket's own lookups carries an own-promotion event
    uint8_t* mstate;         // [n1] CAFE_S_* of the main bucket's last replay
    uint8_t* mark2;          // [n2] 1 = the main pass of this round changed an input of this LRU bucket
    uint8_t* lstate;         // [n2] CAFE_S_* of the LRU bucket's last replay
    // Which buckets replay in a later round: those an input of which changed in the round before.  A main bucket's
    // inputs are the events that land in it (an LRU replay that emits, changes or withdraws one marks the event's
    // target) and the answers its requests for a free row get (the timeline step marks the bucket when an answer
    // is, was or becomes "here is a row"; requests that found the FIFO empty and still do change nothing).  Marks
    // for the next round go to mark_out1 while this round's main pass reads mark_in1 and every bucket clears its
    // own entry there when it has replayed; the engine swaps the two per round.  LRU buckets: mark2 (above) for
    // what the main pass of the same round changed, mark_c2 for the free-row answers, cleared the same way.
    uint8_t* mark_in1;       // [n1]
    uint8_t* mark_out1;      // [n1]
    uint8_t* mark_c2;        // [n2]
    // FIFO timeline believed by this round = the one the previous round produced, as a list of ops
    // (candidate pops and pushes) in op-slot order; the resolve step rewrites it in place
    int32_t* tl_slot;        // [2M] op slot (2p or 2p+1) of every op, ascending
    int32_t* tl_info;        // [2M] 0 = candidate pop, > 0 = push of this hot row
    int32_t* tl_size;        // [2M] FIFO size before the op
    int32_t* tl_rank;        // [2M] successful pops before the op
    int32_t* tl_grp;         // [M / CAFE_TL_GROUP + 2] first op at or after position begin + CAFE_TL_GROUP * g
    int32_t* tl_head;        // [4] number of ops, FIFO size and successful pops after the last op, pushes
    uint32_t* pushbuf;       // [M] pushed rows in op order
    int32_t* tl_blk;         // [2 * blocks] scratch: ops and main-table misses per block of CAFE_TL_BLOCK positions
    CafeFn* tl_agg;          // [blocks of CAFE_TL_BLOCK ops] scratch: composed transfer function per block
    int32_t* nmiss;          // [M] at commit: main-table misses up to and including each position
    // per-lookup results, kept between rounds
    uint8_t* mflag;      // [M] CAFE_F_* written by the main pass
    uint8_t* lflag;      // [M] CAFE_F_* written by the LRU pass for lookups that missed the main table
    int32_t* ins_res;    // [M] result of the event of this position when its target replayed it: 0 ok, -1 failed, >0 failed and pushed this row
    // outputs
    int32_t* mask;       // [M] 1 = this lookup was handed a hot row (the reference's insert result)
    int32_t* post_row;   // [M] hot row of the id at the end of its segment (0 = not hot in the main table)
    CafeRoundResult* res;
};

CAFE_HD float cafe_count_of(const CafeJob& J, int p) { return J.imp ? J.imp[p] : 1.0f; }
CAFE_HD uint32_t cafe_eff_flag(const CafeJob& J, int p) {
    const uint32_t m = J.mflag[p];
    return (m & CAFE_F_MISS) ? ((uint32_t)J.lflag[p] | CAFE_F_MISS) : m;
}

// Believed FIFO size and number of successful pops before op slot `slot`: those before the first op of
// the previous round's list at or after the slot (no op lies in between), or the list's end values.
CAFE_HD void cafe_fifo_before(const CafeJob& J, int64_t slot, int32_t* size, int32_t* rank) {
    if (J.first_round) { *size = J.q_size; *rank = 0; return; }
    const int32_t n = J.tl_head[0];
    const int32_t g = (int32_t)(((slot >> 1) - J.begin) / CAFE_TL_GROUP);
    // first op at or after the slot among the group's ops (up to two per position: binary search)
    int32_t j = J.tl_grp[g], hi = J.tl_grp[g + 1];
    while (j < hi) {
        const int32_t mid = (j + hi) >> 1;
        if ((int64_t)J.tl_slot[mid] < slot) j = mid + 1; else hi = mid;
    }
    if (j < n) { *size = J.tl_size[j]; *rank = J.tl_rank[j]; }
    else { *size = J.tl_head[1]; *rank = J.tl_head[2]; }
}
CAFE_HD bool cafe_fifo_nonempty(const CafeJob& J, int64_t slot) {
    int32_t size, rank;
    cafe_fifo_before(J, slot, &size, &rank);
    return size > 0;
}
// Belief about a pop at op slot `slot`: would the FIFO be non-empty, and which row is at its front.
CAFE_HD bool cafe_would_pop(const CafeJob& J, int64_t slot, int32_t* id) {
    int32_t size, rank;
    cafe_fifo_before(J, slot, &size, &rank);
    *id = 0;
    if (size <= 0) return false;
    if (rank < J.q_size) *id = (int32_t)J.ring[(J.q_head + (uint32_t)rank) & J.ring_mask];
    else if (rank - J.q_size < J.M) *id = (int32_t)J.pushbuf[rank - J.q_size];
    else { CAFE_ATOMIC_OR(&J.res->error, 4); return false; }
    return true;
}

// Smallest event position > after in the chain of bucket events (chains are short; order in the
// chain is arbitrary because it was built with atomic exchanges).
CAFE_HD int cafe_next_event(const CafeJob& J, int head, int after) {
    int best = INT32_MAX;
    for (int e = head; e >= 0; e = J.nxt[e])
        if (e > after && e < best && e < J.limit) best = e;
    return best;
}

// old beliefs of a position; in the first round they are known to be empty (the engine clears the window's
// flags and events before it) and are not read
CAFE_HD uint32_t cafe_old_kind(const CafeJob& J, int p) { return J.first_round ? (uint32_t)CAFE_EV_NONE : J.ev[p].kind; }
CAFE_HD uint32_t cafe_old_mflag(const CafeJob& J, int p) { return J.first_round ? 0u : (uint32_t)J.mflag[p]; }

// ---- between rounds: rebuild the routing of events to the main buckets they land in -----------------
CAFE_HD void cafe_route_position(const CafeJob& J, int p) {
    if (!(J.mflag[p] & CAFE_F_MISS)) return;   // a lookup that hit the main table has no event
    const CafeEvent e = J.ev[p];
    if (e.kind == CAFE_EV_VICTIM) J.nxt[p] = CAFE_ATOMIC_EXCH(&J.head[cafe_hash(e.x, J.n1)], p);
    else if (e.kind == CAFE_EV_OWN) J.mark_own[cafe_hash(e.x, J.n1)] = 1;
}

// the event of position p no longer exists (its lookup hits the main table now, or its LRU replay produces none):
// the main bucket it would have landed in replays without it
CAFE_HD void cafe_withdraw_event(const CafeJob& J, int p) {
    const CafeEvent o = J.ev[p];
    if (o.kind != CAFE_EV_NONE) J.mark_out1[cafe_hash(o.x, J.n1)] = 1;
    J.ev[p].kind = CAFE_EV_NONE;
    J.res->changed = 1;
}

// A job that is shortened to [begin, limit) after a round (a threshold re-fit falls due inside it) keeps what the
// rounds so far worked out for the buckets that saw none of the dropped lookups.  The others replay in the next round:
// the main bucket of every dropped lookup, its LRU bucket if it went there, and the main bucket its event was headed for.
// `mark_next1` is the array the next round's main pass reads.
CAFE_HD void cafe_mark_cut_position(const CafeJob& J, int p, uint8_t* mark_next1) {
    const uint32_t x = J.gid[p];
    mark_next1[cafe_hash(x, J.n1)] = 1;
    if (J.mflag[p] & CAFE_F_MISS) {
        J.mark_c2[cafe_hash(x, J.n2)] = 1;
        const CafeEvent e = J.ev[p];
        if (e.kind != CAFE_EV_NONE) mark_next1[cafe_hash(e.x, J.n1)] = 1;
    }
}

// ---- round step 1: one main bucket ---------------------------------------------------------------
// The replay of a bucket is a small state machine fed one own lookup at a time (feed), so that the
// same code serves a thread that walks its bucket's lookups alone and a warp that loads a long
// bucket's lookups together and hands them to the owning lane.
//
// Between rounds a bucket is replayed again only if something it depends on can have changed: it
// receives events, one of its ids is waiting for a free row (so the FIFO timeline matters), or it was
// in one of these cases in its previous replay (one more replay returns it to the belief-free result).
#define CAFE_CAND 4
struct CafeMainReplay {
    CafeMainBucket b;
    int k, evhead, p_ev;
    bool touched, cand, cond_now, dirty;
    // used by the final pass only (post_row): segment bookkeeping
    int seg_end, i_first, i_cur, ncand;
    int cand_p[CAFE_CAND];
    uint32_t cand_x[CAFE_CAND];

    // does bucket k have to be replayed in this (not first) round?  `cond` receives whether events land in it.
    static CAFE_HD bool wanted(const CafeJob& J, int k, bool* cond) {
        const uint32_t st = J.mstate[k];
        *cond = J.head[k] >= 0 || J.mark_own[k] != 0;   // events land here
        return J.final_pass ? (st & CAFE_S_DIRTY) != 0 : (J.all_active || J.mark_in1[k] != 0);
    }
    // returns false if the bucket does not need to be replayed this round; `pre` = the bucket's batch-start
    // image if the caller has loaded it already
    CAFE_HD bool init(const CafeJob& J, int k_, int i_start, const CafeMainBucket* pre = nullptr) {
        k = k_;
        cond_now = false;
        if (!J.first_round && !wanted(J, k, &cond_now)) return false;
        b = pre ? *pre : J.main_in[k];
        evhead = J.first_round ? -1 : J.head[k];
        p_ev = (evhead < 0) ? INT32_MAX : cafe_next_event(J, evhead, -1);
        touched = cand = dirty = false;
        seg_end = J.seg_off[1];
        i_first = i_cur = i_start;
        ncand = 0;
        return true;
    }
    CAFE_HD void set(int slot, uint32_t v, float c, int32_t d) {
#pragma unroll
        for (int q = 0; q < CAFE_SLOTS; ++q) if (q == slot) { b.val[q] = v; b.cnt[q] = c; b.dic[q] = d; }
    }
    CAFE_HD void note_cand(int p, uint32_t x) {
#pragma unroll
        for (int q = 0; q < CAFE_CAND; ++q) if (q == ncand) { cand_p[q] = p; cand_x[q] = x; }
        ++ncand;
    }
    // final pass: the segment (one field's call) ended: record what a query at this point would return
    CAFE_HD void close_segment(const CafeJob& J) {
        if (dirty) {
            if (ncand <= CAFE_CAND) {
#pragma unroll
                for (int j = 0; j < CAFE_CAND; ++j) if (j < ncand) J.post_row[cand_p[j]] = cafe_probe_hot(b, cand_x[j]);
            } else {
                for (int j = i_first; j < i_cur; ++j) { int q = J.ord1[j]; J.post_row[q] = cafe_probe_hot(b, J.gid[q]); }
            }
        }
        dirty = false; ncand = 0; i_first = i_cur;
    }
    CAFE_HD void enter(const CafeJob& J, int p) {
        if (J.final_pass && p >= seg_end) {
            close_segment(J);
            int s = 0;
            while (p >= J.seg_off[s + 1]) ++s;
            seg_end = J.seg_off[s + 1];
        }
        if (!touched) { cafe_touch(b, J.gflip); touched = true; }
    }
    // the event of position p lands in this bucket (Insert, sketch.cpp:232-259)
    CAFE_HD void apply_event(const CafeJob& J, int p) {
        const CafeEvent e = J.ev[p];
        if (e.kind != CAFE_EV_OWN && e.kind != CAFE_EV_VICTIM) return;   // withdrawn while this pass ran
        int32_t pushed;
        const int ok = cafe_promote(b, e.x, e.cnt, e.dic, &pushed);
        if (!J.final_pass) J.ins_res[p] = ok ? 0 : (pushed != 0 ? pushed : -1);
        dirty = true;
    }
    // believed victim promotions (sketch.cpp:193-195 -> Insert) landing here at positions < before
    CAFE_HD void drain_events(const CafeJob& J, int before) {
        while (p_ev < before) {
            enter(J, p_ev);
            apply_event(J, p_ev);
            p_ev = cafe_next_event(J, evhead, p_ev);
        }
    }
    // own lookup at position p (ascending); a lookup's probe comes before an event of the same position.
    // old_kind / old_flag = what the previous round left for p (cafe_old_kind, cafe_old_mflag).
    CAFE_HD void feed(const CafeJob& J, int p, uint32_t x, float c, uint32_t old_kind, uint32_t old_flag) {
        if (p_ev < p) drain_events(J, p);
        enter(J, p);
        int s = -1;
#pragma unroll
        for (int q = CAFE_SLOTS - 1; q >= 0; --q) if (b.val[q] == x) s = q;
        if (s >= 0) {   // insert(): hit in the main table (sketch.cpp:215-228)
            float cnt0 = 0.f;
            int32_t dic0 = 0;
#pragma unroll
            for (int q = 0; q < CAFE_SLOTS; ++q) if (q == s) { cnt0 = b.cnt[q]; dic0 = b.dic[q]; }
            const float cn = cnt0 + c;
            uint32_t nf = 0;
            if (cn >= J.thr && cn - c < J.thr) nf |= CAFE_F_CROSS;
            if (cn >= J.thr && dic0 == 0) {
                cand = true;
                nf |= CAFE_F_POP0;   // candidate pop at op slot 2p
                int32_t id;
                if (cafe_would_pop(J, 2 * (int64_t)p, &id)) {
                    dic0 = id; nf |= CAFE_F_GOT; dirty = true;
                    if (J.final_pass) note_cand(p, x);
                }
            }
            set(s, x, cn, dic0);
            if (!J.final_pass) {
                // flags and events of the job's window are zero before the first round, so a plain hit
                // (no flag set) has nothing to store then; later rounds store what changed
                if (nf != old_flag) J.mflag[p] = (uint8_t)nf;
                if (!J.first_round) {
                    if (old_kind != CAFE_EV_NONE) cafe_withdraw_event(J, p);
                    if (old_flag & CAFE_F_MISS) { J.mark2[cafe_hash(x, J.n2)] = 1; J.res->miss_changed = 1; }   // its LRU bucket loses this visitor
                }
            }
        } else {
            // final pass: only a lookup that was handed a row (in the LRU stage) needs its post-insert row
            if (J.final_pass) { if (J.lflag[p] & CAFE_F_GOT) note_cand(p, x); }
            else {
                if (old_flag != CAFE_F_MISS) J.mflag[p] = CAFE_F_MISS;   // goes to the LRU stage; that pass writes lflag
                if (!J.first_round && !(old_flag & CAFE_F_MISS)) { J.mark2[cafe_hash(x, J.n2)] = 1; J.res->miss_changed = 1; }   // new visitor
            }
            if (old_kind == CAFE_EV_OWN) {   // believed: this lookup promotes its own id into this bucket
                apply_event(J, p);
                if (!J.final_pass) J.mark2[cafe_hash(x, J.n2)] = 1;   // the LRU bucket reads ins_res[p]
            }
        }
        ++i_cur;
    }
    CAFE_HD void finish(const CafeJob& J) {
        drain_events(J, INT32_MAX);
        if (J.final_pass) { close_segment(J); return; }
        J.mstate[k] = (uint8_t)((cond_now ? CAFE_S_COND : 0) | (cand ? CAFE_S_CAND : 0) | (dirty ? CAFE_S_DIRTY : 0));
        J.mark_in1[k] = 0;
        J.main_out[k] = b;
    }
};

CAFE_HD void cafe_main_pass_bucket(const CafeJob& J, int k) {
    CafeMainReplay R;
    const int iend = J.start1[k + 1];
    int i = J.beg1[k];
    if (!R.init(J, k, i)) return;
    for (; i < iend; ++i) {
        const int p = J.ord1[i];
        if (p >= J.limit) break;
        R.feed(J, p, J.gid[p], cafe_count_of(J, p), cafe_old_kind(J, p), cafe_old_mflag(J, p));
    }
    R.finish(J);
}

// ---- round step 2: one LRU bucket (insertLRU, sketch.cpp:161-210) ---------------------------------
// LRU clock values are written as t0 + 1 + position while the rounds run (monotone in the order of
// visits and above every stamp of the batch-start state, which is all the replay needs); they are
// turned into the reference's consecutive numbering at commit (cafe_lru_tconvert).
struct CafeLruReplay {
    CafeLruBucket b;
    int k, n_ev;
    bool touched, cand, cond_now;

    static CAFE_HD bool wanted(const CafeJob& J, int k, bool* cond) {
        const uint32_t st = J.lstate[k];
        *cond = J.mark2[k] != 0;
        (void)st;
        return J.all_active || *cond || J.mark_c2[k] != 0;
    }
    CAFE_HD bool init(const CafeJob& J, int k_, const CafeLruBucket* pre = nullptr) {
        k = k_;
        cond_now = false;
        if (!J.first_round && !wanted(J, k, &cond_now)) return false;
        b = pre ? *pre : J.lru_in[k];
        n_ev = 0;
        touched = cand = false;
        return true;
    }
    CAFE_HD void set(int slot, uint32_t v, float c, int32_t d, int32_t tt) {
#pragma unroll
        for (int q = 0; q < CAFE_SLOTS; ++q) if (q == slot) { b.val[q] = v; b.cnt[q] = c; b.dic[q] = d; b.t[q] = tt; }
    }
    // `pre_ev` / `pre_ins`: the event and the ins_res the previous round left for this position, if the caller has
    // loaded them already (a warp loads them for 32 misses at once); null = read here
    CAFE_HD void emit(const CafeJob& J, int p, uint32_t kind, uint32_t x, float cnt, int32_t dic, const CafeEvent* pre_ev) {
        if (J.first_round) {
            if (kind == CAFE_EV_NONE) return;   // events of the window are cleared before the first round
            J.res->changed = 1;
        } else {
            const CafeEvent o = pre_ev ? *pre_ev : J.ev[p];
            bool same;
            if (kind == CAFE_EV_NONE) same = (o.kind == CAFE_EV_NONE);
            else same = (o.kind == kind && o.x == x && o.dic == dic && cafe_float_bits(o.cnt) == cafe_float_bits(cnt));
            if (same) return;
            J.res->changed = 1;
            if (o.kind != CAFE_EV_NONE) J.mark_out1[cafe_hash(o.x, J.n1)] = 1;   // the old event's target loses it
            if (kind == CAFE_EV_NONE) { J.ev[p].kind = CAFE_EV_NONE; return; }
        }
        J.mark_out1[cafe_hash(x, J.n1)] = 1;   // the new event's target
        CafeEvent e;
        e.x = x; e.cnt = cnt; e.dic = dic; e.kind = kind;
        J.ev[p] = e;
    }
    // a lookup at position p (ascending) that missed the main table
    CAFE_HD void feed(const CafeJob& J, int p, uint32_t x, float c, const CafeEvent* pre_ev = nullptr,
                      const int32_t* pre_ins = nullptr) {
        if (!touched) { cafe_touch(b, J.gflip); touched = true; }
        const int32_t tp = J.t0 + 1 + p;
        int hit = -1, vic = -1, t_min = 1000000000;
#pragma unroll
        for (int q = 0; q < CAFE_SLOTS; ++q) {
            if (hit < 0) {
                if (b.val[q] == x) hit = q;
                else if (t_min > b.t[q]) { t_min = b.t[q]; vic = q; }
            }
        }
        uint32_t nf = 0;
        if (hit >= 0) {
            float cnt0 = 0.f;
            int32_t dic0 = 0;
#pragma unroll
            for (int q = 0; q < CAFE_SLOTS; ++q) if (q == hit) { cnt0 = b.cnt[q]; dic0 = b.dic[q]; }
            const float cn = cnt0 + c;
            if (cn >= J.thr && cn - c < J.thr) nf |= CAFE_F_CROSS;
            if (cn >= J.thr && dic0 == 0) {
                cand = true;
                nf |= CAFE_F_POP0;   // candidate pop at op slot 2p (before the possible push-back at 2p+1)
                int32_t id;
                if (cafe_would_pop(J, 2 * (int64_t)p, &id)) { dic0 = id; nf |= CAFE_F_GOT; }
            }
            if (cn >= J.thr) {
                ++n_ev;
                emit(J, p, CAFE_EV_OWN, x, cn, dic0, pre_ev);
                // the main pass of this round replayed the event this position carried before the round
                if (!J.first_round && (pre_ins ? *pre_ins : J.ins_res[p]) != 0) nf &= ~(uint32_t)CAFE_F_GOT;
                set(hit, 0u, 0.0f, 0, 0);   // the slot is cleared whether or not the promotion succeeded
            } else {
                set(hit, x, cn, dic0, tp);
                emit(J, p, CAFE_EV_NONE, 0, 0.0f, 0, pre_ev);
            }
        } else {
            if (vic < 0) { CAFE_ATOMIC_OR(&J.res->error, 2); vic = 0; }
            uint32_t vval = 0;
            float vcnt = 0.f;
            int32_t vdic = 0;
#pragma unroll
            for (int q = 0; q < CAFE_SLOTS; ++q) if (q == vic) { vval = b.val[q]; vcnt = b.cnt[q]; vdic = b.dic[q]; }
            if (vdic != 0 || vcnt >= 5.0f) {
                ++n_ev;
                emit(J, p, CAFE_EV_VICTIM, vval, vcnt, vdic, pre_ev);
            } else {
                emit(J, p, CAFE_EV_NONE, 0, 0.0f, 0, pre_ev);
            }
            int32_t ndic = 0;
            if (1.0f >= J.thr && 1.0f - c < J.thr) nf |= CAFE_F_CROSS;
            if (1.0f >= J.thr) {
                cand = true;
                nf |= CAFE_F_POP1;   // candidate pop at op slot 2p+1 (after the victim's possible push-back at 2p)
                int32_t id;
                if (cafe_would_pop(J, 2 * (int64_t)p + 1, &id)) { ndic = id; nf |= CAFE_F_GOT; }
            }
            set(vic, x, 1.0f, ndic, tp);
        }
        J.lflag[p] = (uint8_t)nf;
    }
    CAFE_HD void finish(const CafeJob& J) {
        if (n_ev) CAFE_ATOMIC_ADD(&J.res->n_events, n_ev);
        J.lstate[k] = (uint8_t)((cond_now ? CAFE_S_COND : 0) | (cand ? CAFE_S_CAND : 0));
        J.mark_c2[k] = 0;
        J.lru_out[k] = b;
    }
};

CAFE_HD void cafe_lru_pass_bucket(const CafeJob& J, int k) {
    CafeLruReplay R;
    if (!R.init(J, k)) return;
    const int jend = J.start2[k + 1];
    for (int j = J.beg2[k]; j < jend; ++j) {
        const int p = J.ord2[j];
        if (p >= J.limit) break;
        if (!(J.mflag[p] & CAFE_F_MISS)) continue;
        R.feed(J, p, J.gid[p], cafe_count_of(J, p));
    }
    R.finish(J);
}

// at commit: first entry of a bucket's sorted lookups that lies at or beyond `limit` (positions ascend)
CAFE_HD int32_t cafe_advance_cursor(const int32_t* ord, int32_t lo, int32_t hi, int32_t limit) {
    while (lo < hi) {
        const int32_t mid = (lo + hi) >> 1;
        if (ord[mid] < limit) lo = mid + 1; else hi = mid;
    }
    return lo;
}
// at commit: LRU clock values written as t0 + 1 + position become t0 + (rank of the visit)
CAFE_HD void cafe_lru_tconvert(const CafeJob& J, int k) {
    CafeLruBucket& b = J.lru_out[k];
#pragma unroll
    for (int q = 0; q < CAFE_SLOTS; ++q)
        if (b.t[q] > J.t0) b.t[q] = J.t0 + J.nmiss[b.t[q] - J.t0 - 1];   // misses up to and including that position
}
// at commit: the reference's per-lookup insert result
CAFE_HD void cafe_finalize_position(const CafeJob& J, int p) {
    J.mask[p] = (cafe_eff_flag(J, p) & CAFE_F_GOT) ? 1 : 0;
}

// ---- round step 3: the FIFO timeline ---------------------------------------------------------------
// Each position owns two op slots (2p, 2p+1).  An op is a candidate pop or a push; the FIFO size
// evolves as s -> max(s + a, b) per op (pop: a=-1,b=0; push: a=+1,b=-inf), a family closed under
// composition, so sizes come from one scan; the number of successful pops before an op follows from
// size = q_size + pushes - pops.  Few positions carry an op, so the ops are first compacted into a
// list (count per block of positions, then emit at the block's offset) and only the list is scanned.
#define CAFE_NEG_INF (-(1 << 29))
struct CafeOps { int op0, op1; int32_t id0, id1; };   // op: 0 none, 1 pop, 2 push

CAFE_HD CafeOps cafe_ops_of(const CafeJob& J, int p) {
    CafeOps o; o.op0 = o.op1 = 0; o.id0 = o.id1 = 0;
    const uint32_t f = cafe_eff_flag(J, p);
    if (f & CAFE_F_POP0) o.op0 = 1;
    if (f & CAFE_F_POP1) o.op1 = 1;
    const int32_t r = (J.first_round || !(f & CAFE_F_MISS)) ? 0 : J.ins_res[p];
    if (r > 0) {
        // the event of this position failed at its target and pushed its row back: after the pop for an
        // own promotion (slot 2p+1), before the pop for a victim promotion (slot 2p)
        const uint32_t kind = J.ev[p].kind;
        if (kind == CAFE_EV_OWN) { if (o.op1 == 0) { o.op1 = 2; o.id1 = r; } else J.res->changed = 1; }
        else if (kind == CAFE_EV_VICTIM) { if (o.op0 == 0) { o.op0 = 2; o.id0 = r; } else J.res->changed = 1; }
    }
    return o;
}
CAFE_HD int cafe_ops_count(const CafeOps& o) { return (o.op0 != 0) + (o.op1 != 0); }
// (a2,b2) after (a1,b1)
CAFE_HD void cafe_compose(int32_t a1, int32_t b1, int32_t a2, int32_t b2, int32_t* a, int32_t* b) {
    int32_t bb = b1 + a2;
    if (bb < CAFE_NEG_INF) bb = CAFE_NEG_INF;
    *a = a1 + a2;
    *b = bb > b2 ? bb : b2;
}
CAFE_HD CafeFn cafe_fn_identity() { CafeFn f; f.a = 0; f.b = CAFE_NEG_INF; f.np = 0; f.pad = 0; return f; }
CAFE_HD CafeFn cafe_fn_then(const CafeFn& f, const CafeFn& g) {   // g after f
    CafeFn r;
    cafe_compose(f.a, f.b, g.a, g.b, &r.a, &r.b);
    r.np = f.np + g.np;
    r.pad = 0;
    return r;
}
CAFE_HD int32_t cafe_apply_fn(int32_t a, int32_t b, int32_t s) { int32_t v = s + a; return v > b ? v : b; }
// transfer function of one list entry
CAFE_HD CafeFn cafe_fn_of_info(int32_t info) {
    CafeFn f;
    if (info == 0) { f.a = -1; f.b = 0; f.np = 0; }
    else { f.a = 1; f.b = CAFE_NEG_INF; f.np = 1; }
    f.pad = 0;
    return f;
}
// 3a: ops of position p go to list entries j, j+1, ...; the list is updated in place, and an entry that
// differs from what the previous round left there means the timeline this round consumed has changed
// (the first round consumed none: its change test is in cafe_tl_finish_op)
CAFE_HD void cafe_tl_emit(const CafeJob& J, int p, const CafeOps& o, int32_t j, int32_t n_old) {
    bool diff = false;
    if (o.op0 != 0) {
        const int32_t slot = 2 * p, info = o.op0 == 2 ? o.id0 : 0;
        if (!J.first_round && (j >= n_old || J.tl_slot[j] != slot || J.tl_info[j] != info)) diff = true;
        J.tl_slot[j] = slot; J.tl_info[j] = info;
        ++j;
    }
    if (o.op1 != 0) {
        const int32_t slot = 2 * p + 1, info = o.op1 == 2 ? o.id1 : 0;
        if (!J.first_round && (j >= n_old || J.tl_slot[j] != slot || J.tl_info[j] != info)) diff = true;
        J.tl_slot[j] = slot; J.tl_info[j] = info;
    }
    if (diff) { J.res->changed = 1; J.res->tl_changed = 1; }
}
// after the last position: the list's length (a different length is a change too)
CAFE_HD void cafe_tl_set_count(const CafeJob& J, int32_t n_new, int32_t n_old) {
    if (!J.first_round && n_new != n_old) { J.res->changed = 1; J.res->tl_changed = 1; }
    J.tl_head[0] = n_new;
    if (n_new == 0) { J.tl_head[1] = J.q_size; J.tl_head[2] = 0; J.tl_head[3] = 0; J.res->n_pop_ok = 0; J.res->n_push = 0; }
}
// 3b: list entry j of n, given the composition `before` of all entries ahead of it
CAFE_HD void cafe_tl_finish_op(const CafeJob& J, int32_t j, int32_t n, const CafeFn& before) {
    const int32_t info = J.tl_info[j];
    const int32_t s = cafe_apply_fn(before.a, before.b, J.q_size);
    const int32_t rank = J.q_size + before.np - s;
    J.tl_size[j] = s;
    J.tl_rank[j] = rank;
    if (info != 0) J.pushbuf[before.np] = (uint32_t)info;
    else {
        // a request for a free row: its bucket has to replay next round unless the answer was "none" and still is
        const int p = J.tl_slot[j] >> 1;
        const uint32_t f = cafe_eff_flag(J, p);
        if (s > 0 || (f & CAFE_F_GOT)) {
            if (f & CAFE_F_MISS) J.mark_c2[cafe_hash(J.gid[p], J.n2)] = 1;
            else J.mark_out1[cafe_hash(J.gid[p], J.n1)] = 1;
        }
    }
    // the first round believed an untouched FIFO everywhere: a push or a successful pop contradicts that
    if (J.first_round && (info != 0 || s > 0)) { J.res->changed = 1; J.res->tl_changed = 1; }
    if (j == n - 1) {
        const CafeFn after = cafe_fn_then(before, cafe_fn_of_info(info));
        const int32_t s_end = cafe_apply_fn(after.a, after.b, J.q_size);
        const int32_t pops = J.q_size + after.np - s_end;
        J.tl_head[1] = s_end; J.tl_head[2] = pops; J.tl_head[3] = after.np;
        J.res->n_pop_ok = pops;
        J.res->n_push = after.np;
    }
}

// 3d: what position p adds to the per-segment change of real_n (a threshold crossing, sketch.cpp:169,
// 200, 218) and to the number of LRU visits
CAFE_HD void cafe_position_counts(const CafeJob& J, int p, int* crossed, int* missed) {
    const uint32_t f = cafe_eff_flag(J, p);
    *crossed = (f & CAFE_F_CROSS) ? 1 : 0;
    *missed = (f & CAFE_F_MISS) ? 1 : 0;
}
CAFE_HD int cafe_segment_of(const CafeJob& J, int p) {
    int lo = 0, hi = J.nseg - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (p >= J.seg_off[mid + 1]) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// ---- commit of the FIFO after a converged round: live pushes go into the ring ----------------------
// Entry j of the round's push list has virtual rank q_size + j; ranks below n_pop_ok were consumed.
CAFE_HD void cafe_commit_push(uint32_t* ring, uint32_t ring_mask, uint32_t q_head, int32_t q_size,
                              int32_t n_pop_ok, const uint32_t* pushbuf, int j) {
    int64_t rank = (int64_t)q_size + j;
    if (rank >= n_pop_ok) ring[(q_head + (uint32_t)rank) & ring_mask] = pushbuf[j];
}

// =================================================================================================
// Threshold re-fit (reset, sketch.cpp:76-116) helpers.  Candidates are numbered canonically: main
// slots first (bucket-major), then LRU slots.
// =================================================================================================
CAFE_HD int cafe_reset_touch_count_main(CafeMainBucket& b, uint32_t gflip, float thr) {
    cafe_touch(b, gflip);
    int n = 0;
#pragma unroll
    for (int i = 0; i < CAFE_SLOTS; ++i) n += (b.cnt[i] >= thr || b.dic[i] != 0);
    return n;
}
CAFE_HD int cafe_reset_touch_count_lru(CafeLruBucket& b, uint32_t gflip, float thr) {
    cafe_touch(b, gflip);
    int n = 0;
#pragma unroll
    for (int i = 0; i < CAFE_SLOTS; ++i) n += (b.cnt[i] >= thr || b.dic[i] != 0);
    return n;
}
CAFE_HD int32_t* cafe_slot_dic(CafeMainBucket* mb, CafeLruBucket* lb, int32_t n1, int32_t order) {
    const int32_t main_slots = n1 * CAFE_SLOTS;
    if (order < main_slots) return &mb[order >> 2].dic[order & 3];
    order -= main_slots;
    return &lb[order >> 2].dic[order & 3];
}
