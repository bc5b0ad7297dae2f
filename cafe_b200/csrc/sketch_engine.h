// sketch_engine.h -- host-side driver of the device-resident HotSketch.
//
// SketchEngine<Backend> owns the sketch state (two images of each bucket table, the free-row FIFO
// ring, the scalars the reference keeps in class members and file-scope globals) and the workspace
// of the parallel insert, and sequences the rounds, the call-boundary work (decay clock, flip bit,
// threshold re-fit) and the commit.  The Backend supplies memory and the per-bucket / per-position
// passes: the CUDA backend launches kernels, the host backend (tests only) runs the same functions
// in loops.  Scalars live on the host; kernels receive them by value.
//
// Reference semantics reproduced here: batch_insert / batch_insert_val prologue
// (tricks/sketch.cpp:266-275, 281-291), reset (:76-116), init (:309-313).
#pragma once
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "sketch_core.cuh"

struct CafeSketchStats {
    int64_t calls, lookups, rounds, jobs, truncated_jobs, resets, resets_refused, flips;
    int64_t seq_fallbacks, main_hits, lru_visits, events, max_rounds;
};

template <class BE>
class SketchEngine {
public:
    // scalars (sketch.cpp:16-21 and the globals of :7-13)
    int lim = 0, n1 = 0, n2 = 0, adjust = 1;
    float thr = 0.f;
    int real_n = 0, num = 0, t = 0;
    uint32_t gflip = 0;
    double alpha = 1.0, decay_importance = 1.0;
    int batch_num = 0;
    uint32_t q_head = 0;
    int q_size = 0;
    uint32_t ring_mask = 0;
    int round_cap = 48;
    double cross_rate = -1.0;         // threshold crossings per lookup seen in recent jobs (-1: unknown)
    int window = CAFE_MAX_SEGMENTS;   // upper bound on the segments fused into one job
    bool size_jobs_by_rate = true;    // end a job where the crossing rate predicts the next re-fit (off: tests of the cut path)
    int last_status = CAFE_OK;
    CafeSketchStats stats;

    BE be;

    SketchEngine() { memset(&stats, 0, sizeof(stats)); }
    ~SketchEngine() { release(); }

    int init(int lim_, float thr_, int adjust_, double alpha_, int max_lookups) {
        release();
        if (lim_ < 20 || max_lookups < 1) return CAFE_ERR_ARG;
        lim = lim_; thr = thr_; adjust = adjust_; alpha = alpha_;
        n1 = (int)(lim * 0.9);   // sketch.cpp:51-52
        n2 = (int)(lim * 0.1);
        if (n1 < 1 || n2 < 1) return CAFE_ERR_ARG;
        real_n = num = t = 0; gflip = 0; decay_importance = 1.0; batch_num = 0;
        cap = max_lookups;
        uint32_t rc = 1;
        while (rc < (uint32_t)lim + 1) rc <<= 1;
        ring_mask = rc - 1;
        for (int i = 0; i < 2; ++i) {
            mainb[i] = (CafeMainBucket*)be.alloc(sizeof(CafeMainBucket) * (size_t)n1);
            lrub[i] = (CafeLruBucket*)be.alloc(sizeof(CafeLruBucket) * (size_t)n2);
            if (!mainb[i] || !lrub[i]) return CAFE_ERR_CUDA;
        }
        be.memset(mainb[0], 0, sizeof(CafeMainBucket) * (size_t)n1);
        be.memset(lrub[0], 0, sizeof(CafeLruBucket) * (size_t)n2);
        cur = 0;
        ring = (uint32_t*)be.alloc(sizeof(uint32_t) * (size_t)rc);
        if (!ring) return CAFE_ERR_CUDA;
        be.fill_iota(ring, lim - 1, 1);   // free rows 1..lim-1 (sketch.cpp:55-56); row 0 is never handed out
        q_head = 0; q_size = lim - 1;
        // workspace of the parallel insert
        size_t M = (size_t)cap;
        ord1 = (int32_t*)be.alloc(4 * M); ord2 = (int32_t*)be.alloc(4 * M);
        sgid1 = (uint32_t*)be.alloc(4 * M); sgid2 = (uint32_t*)be.alloc(4 * M);
        simp1 = (float*)be.alloc(4 * M); simp2 = (float*)be.alloc(4 * M);
        start1 = (int32_t*)be.alloc(4 * ((size_t)n1 + 1)); start2 = (int32_t*)be.alloc(4 * ((size_t)n2 + 1));
        beg1 = (int32_t*)be.alloc(4 * (size_t)n1); beg2 = (int32_t*)be.alloc(4 * (size_t)n2);
        ev = (CafeEvent*)be.alloc(sizeof(CafeEvent) * M);
        head = (int32_t*)be.alloc(4 * (size_t)n1);
        nxt = (int32_t*)be.alloc(4 * M);
        // mark_own | mark2 | round result: contiguous so that one memset clears what a round needs cleared
        off_mark2 = ((size_t)n1 + 63) & ~(size_t)63;
        off_res = (off_mark2 + (size_t)n2 + 63) & ~(size_t)63;
        span_clear = off_res + sizeof(CafeRoundResult);
        mark_own = (uint8_t*)be.alloc(span_clear);
        mark2 = mark_own ? mark_own + off_mark2 : nullptr;
        res_dev = mark_own ? (CafeRoundResult*)(mark_own + off_res) : nullptr;
        mstate = (uint8_t*)be.alloc((size_t)n1);
        lstate = (uint8_t*)be.alloc((size_t)n2);
        mark_w1[0] = (uint8_t*)be.alloc(2 * (size_t)n1 + (size_t)n2);
        mark_w1[1] = mark_w1[0] ? mark_w1[0] + n1 : nullptr;
        mark_c2 = mark_w1[0] ? mark_w1[0] + 2 * (size_t)n1 : nullptr;
        if (mark_w1[0]) be.memset(mark_w1[0], 0, 2 * (size_t)n1 + (size_t)n2);
        mark_par = 0;
        mflag = (uint8_t*)be.alloc(M); lflag = (uint8_t*)be.alloc(M);
        tl_slot = (int32_t*)be.alloc(8 * M); tl_info = (int32_t*)be.alloc(8 * M);
        tl_size = (int32_t*)be.alloc(8 * M); tl_rank = (int32_t*)be.alloc(8 * M);
        tl_grp = (int32_t*)be.alloc(4 * (M / CAFE_TL_GROUP + 2));
        tl_head = (int32_t*)be.alloc(4 * 4);
        pushbuf = (uint32_t*)be.alloc(4 * M);
        tl_blk = (int32_t*)be.alloc(4 * 2 * (M / CAFE_TL_BLOCK + 2));
        tl_agg = (CafeFn*)be.alloc(sizeof(CafeFn) * (2 * M / CAFE_TL_BLOCK + 2));
        nmiss = (int32_t*)be.alloc(4 * M);
        ins_res = (int32_t*)be.alloc(4 * M);
        seq_dev = (CafeSeqState*)be.alloc(sizeof(CafeSeqState));
        size_t ncand = (size_t)(n1 + n2) * CAFE_SLOTS;
        cand_key[0] = (uint32_t*)be.alloc(4 * ncand); cand_key[1] = (uint32_t*)be.alloc(4 * ncand);
        cand_val[0] = (int32_t*)be.alloc(4 * ncand); cand_val[1] = (int32_t*)be.alloc(4 * ncand);
        cand_cnt = (int32_t*)be.alloc(4 * ((size_t)n1 + n2 + 1));
        reset_out = (int32_t*)be.alloc(4 * 8);
        if (!be.prepare(cap, n1, n2)) return CAFE_ERR_CUDA;
        if (!ord1 || !ord2 || !start1 || !start2 || !beg1 || !beg2 || !mflag || !lflag || !ev || !head || !nxt || !mark_own || !mstate || !mark2 || !lstate || !ins_res ||
            !res_dev || !seq_dev || !cand_key[0] || !cand_key[1] || !cand_val[0] || !cand_val[1] || !cand_cnt || !reset_out)
            return CAFE_ERR_CUDA;
        if (!sgid1 || !sgid2 || !simp1 || !simp2 || !mark_w1[0]) return CAFE_ERR_CUDA;
        if (!tl_slot || !tl_info || !tl_size || !tl_rank || !tl_grp || !tl_head || !pushbuf || !tl_blk || !tl_agg || !nmiss) return CAFE_ERR_CUDA;
        ready = true;
        return be.ok() ? CAFE_OK : CAFE_ERR_CUDA;
    }

    int capacity() const { return cap; }
    const CafeMainBucket* main_table() const { return mainb[cur]; }
    const CafeLruBucket* lru_table() const { return lrub[cur]; }
    CafeMainBucket* main_table_mut() { return mainb[cur]; }
    CafeLruBucket* lru_table_mut() { return lrub[cur]; }
    const uint32_t* ring_ptr() const { return ring; }

    // batch_query (sketch.cpp:260-265): out[i] = -row if hot else (int)id
    int query(const uint32_t* gid, int n, int32_t* out) {
        if (!ready || n < 0) return CAFE_ERR_ARG;
        if (n == 0) return CAFE_OK;
        be.query(mainb[cur], n1, gid, n, out);
        return be.ok() ? CAFE_OK : CAFE_ERR_CUDA;
    }

    // Starts the bucket sorts of the next insert_segments call early, on the backend's side lanes, for
    // a caller that knows the ids before it knows the counts.  Only honoured when that call passes the
    // same pointer and its whole input is one stretch of n lookups.
    void presort(const uint32_t* gid, int n) {
        presorted_gid = nullptr;
        if (ready) be.sort_join(-1);   // a null gid withdraws an earlier presort
        if (!ready || !gid || n <= 0 || n > cap) return;
        be.sort_lookups(gid, n, n1, ord1, sgid1, start1, beg1, 1);
        be.sort_lookups(gid, n, n2, ord2, sgid2, start2, beg2, 2);
        presorted_gid = gid; presorted_n = n;
    }

    // The next insert_segments call may use the counts of segments >= seg only after the backend's gate
    // event has fired on its stream (the caller is still producing them); -1 = no gate.
    void set_gate(int seg) { gate_seg = seg; }

    // One batch_insert_val call per segment, in order (imp == null: batch_insert, unit counts).
    // mask[p] = the reference's per-lookup result; post_row[p] (optional) = hot row a query would
    // return for the id right after its own segment's call (0 = none).  parallel=false runs the
    // sequential kernel for every segment.
    int insert_segments(const uint32_t* gid, const float* imp, const int* seg_off, int nseg, int32_t* mask,
                        int32_t* post_row, bool parallel) {
        if (!ready || nseg < 1 || !seg_off || seg_off[0] != 0) return CAFE_ERR_ARG;
        for (int s = 0; s < nseg; ++s) if (seg_off[s + 1] < seg_off[s]) return CAFE_ERR_ARG;
        const int total = seg_off[nseg];
        if (total > 0 && (!gid || !mask)) return CAFE_ERR_ARG;
        last_status = CAFE_OK;
        struct GateReset { int& g; ~GateReset() { g = -1; } } gate_reset{gate_seg};
        if (gate_seg >= nseg) gate_seg = -1;
        int s = 0;
        while (s < nseg) {
            // a stretch of calls whose lookups fit the workspace is sorted by bucket once
            int se = s;
            while (se < nseg && seg_off[se + 1] - seg_off[s] <= cap) ++se;
            if (se == s) return CAFE_ERR_CAPACITY;
            const int base = seg_off[s];
            const int mtot = seg_off[se] - base;
            const uint32_t* g = gid ? gid + base : nullptr;
            const float* im = imp ? imp + base : nullptr;
            int32_t* mk = mask ? mask + base : nullptr;
            int32_t* pr = post_row ? post_row + base : nullptr;
            struct SortJoin { BE& be; ~SortJoin() { be.sort_join(-1); } } sort_join_guard{be};
            if (parallel && mtot > 0 && !(presorted_gid == g && presorted_n == mtot)) {
                be.sort_join(-1);   // a head start for other arrays may still be writing the orders
                // the LRU table's order is first needed by the first LRU pass: it is built on a side
                // lane of the backend while the main table's order and first pass proceed
                be.sort_lookups(g, mtot, n2, ord2, sgid2, start2, beg2, 2);
                be.sort_lookups(g, mtot, n1, ord1, sgid1, start1, beg1, 0);
            }
            presorted_gid = nullptr;
            if (parallel && mtot > 0 && im) {   // counts in the two bucket orders, beside the sorted positions and ids
                if (gate_seg >= 0) { be.wait_gate(); gate_seg = -1; }   // every count must exist before it is permuted
                be.sort_join(-1);
                be.gather_counts(im, ord1, ord2, mtot, simp1, simp2);
            }
            while (s < se) {
                // counts of the calls from gate_seg on become valid only when the caller's gate opens
                if (gate_seg >= 0 && s >= gate_seg) { be.wait_gate(); gate_seg = -1; }
                call_boundary();
                if (last_status == CAFE_ERR_CUDA) return last_status;
                int e = s + 1;
                if (parallel) {
                    // fuse following calls while their boundaries are known to be uneventful: the decay
                    // clock is deterministic, the re-fit condition is checked after the fact
                    double d = decay_importance;
                    int maxe = std::min(se, s + std::max(1, std::min(window, (int)CAFE_MAX_SEGMENTS)));
                    if (gate_seg >= 0 && s < gate_seg) maxe = std::min(maxe, gate_seg);   // a job ends at the gate
                    while (e < maxe) {
                        double d2 = d * alpha;
                        if (d2 > CAFE_DECAY_BASE) break;
                        // stop where a threshold re-fit is expected (the exact test runs on the results)
                        if (adjust && size_jobs_by_rate && cross_rate >= 0 &&
                            real_n + cross_rate * ((double)seg_off[e] - seg_off[s]) > lim * 1.2) break;
                        d = d2; ++e;
                    }
                }
                int done_e = e;
                const int lo = seg_off[s] - base, hi = seg_off[e] - base;
                if (hi > lo) {
                    if (parallel) {
                        int rel[CAFE_MAX_SEGMENTS + 1];
                        for (int i = 0; i <= e - s; ++i) rel[i] = seg_off[s + i] - base;
                        int done = 0;
                        int rc = run_parallel(g, im, mtot, rel, e - s, mk, pr, &done);
                        if (rc != CAFE_OK) return rc;
                        done_e = s + done;
                        const int upto = seg_off[done_e] - base;
                        be.sort_join(-1);
                        if (!cursors_advanced) {   // (the commit of a converged job moves them itself)
                            be.advance_cursors(ord1, start1, beg1, n1, upto);
                            be.advance_cursors(ord2, start2, beg2, n2, upto);
                        }
                    } else {
                        int rc = run_sequential(g + lo, im ? im + lo : nullptr, hi - lo, mk + lo, pr ? pr + lo : nullptr);
                        if (rc != CAFE_OK) return rc;
                    }
                }
                // boundaries inside the fused range: nothing happens at them except the clocks
                for (int b = s + 1; b < done_e; ++b) { ++batch_num; decay_importance *= alpha; ++stats.calls; }
                s = done_e;
            }
        }
        stats.lookups += total;
        if (!be.ok()) return last_status = CAFE_ERR_CUDA;
        return last_status;
    }

    // reset() of the reference, callable directly for tests.
    int refit_threshold() {
        int32_t l = 0;
        be.reset_collect(mainb[cur], lrub[cur], n1, n2, gflip, thr, cand_cnt, cand_key[0], cand_val[0], &l);
        if (!be.ok()) return last_status = CAFE_ERR_CUDA;
        if (l < lim) { ++stats.resets_refused; return last_status = CAFE_ERR_RESET_UNDERFLOW; }
        be.sort_pairs(cand_key[0], cand_val[0], cand_key[1], cand_val[1], l, 32);
        int32_t out[8];
        be.reset_apply(cand_key[1], cand_val[1], l, lim, mainb[cur], lrub[cur], n1, ring, ring_mask, q_head, q_size,
                       reset_out, out);
        if (!be.ok()) return last_status = CAFE_ERR_CUDA;
        uint32_t bits = (uint32_t)out[0];
        memcpy(&thr, &bits, 4);
        const int npush = out[1], npop = out[2];
        q_head += (uint32_t)npop;
        q_size += npush - npop;
        real_n = lim;
        ++stats.resets;
        return CAFE_OK;
    }

    // ---- state export (tests, checkpoints): flat arrays in the oracle's dump layout ----------------
    void dump(uint32_t* mval, float* mcnt, int32_t* mdic, uint8_t* mflip, uint32_t* lval, float* lcnt, int32_t* ldic,
              int32_t* lt, uint8_t* lflip, uint32_t* queue) {
        std::vector<CafeMainBucket> hm((size_t)n1);
        std::vector<CafeLruBucket> hl((size_t)n2);
        std::vector<uint32_t> hr((size_t)ring_mask + 1);
        be.d2h(hm.data(), mainb[cur], sizeof(CafeMainBucket) * (size_t)n1);
        be.d2h(hl.data(), lrub[cur], sizeof(CafeLruBucket) * (size_t)n2);
        be.d2h(hr.data(), ring, 4 * ((size_t)ring_mask + 1));
        for (int k = 0; k < n1; ++k) {
            for (int i = 0; i < 4; ++i) { mval[k * 4 + i] = hm[k].val[i]; mcnt[k * 4 + i] = hm[k].cnt[i]; mdic[k * 4 + i] = hm[k].dic[i]; }
            mflip[k] = (uint8_t)hm[k].flip;
        }
        for (int k = 0; k < n2; ++k) {
            for (int i = 0; i < 4; ++i) { lval[k * 4 + i] = hl[k].val[i]; lcnt[k * 4 + i] = hl[k].cnt[i]; ldic[k * 4 + i] = hl[k].dic[i]; lt[k * 4 + i] = hl[k].t[i]; }
            lflip[k] = (uint8_t)hl[k].flip;
        }
        for (int i = 0; i < q_size; ++i) queue[i] = hr[(q_head + (uint32_t)i) & ring_mask];
    }

    // inverse of dump (restore from a checkpoint)
    int load(const uint32_t* mval, const float* mcnt, const int32_t* mdic, const uint8_t* mflip, const uint32_t* lval,
             const float* lcnt, const int32_t* ldic, const int32_t* lt, const uint8_t* lflip, const uint32_t* queue,
             int qn) {
        if (!ready || qn < 0 || qn > (int)ring_mask) return CAFE_ERR_ARG;
        std::vector<CafeMainBucket> hm((size_t)n1);
        std::vector<CafeLruBucket> hl((size_t)n2);
        std::vector<uint32_t> hr((size_t)ring_mask + 1, 0u);
        memset(hm.data(), 0, sizeof(CafeMainBucket) * (size_t)n1);
        memset(hl.data(), 0, sizeof(CafeLruBucket) * (size_t)n2);
        for (int k = 0; k < n1; ++k) {
            for (int i = 0; i < 4; ++i) { hm[k].val[i] = mval[k * 4 + i]; hm[k].cnt[i] = mcnt[k * 4 + i]; hm[k].dic[i] = mdic[k * 4 + i]; }
            hm[k].flip = mflip[k];
        }
        for (int k = 0; k < n2; ++k) {
            for (int i = 0; i < 4; ++i) { hl[k].val[i] = lval[k * 4 + i]; hl[k].cnt[i] = lcnt[k * 4 + i]; hl[k].dic[i] = ldic[k * 4 + i]; hl[k].t[i] = lt[k * 4 + i]; }
            hl[k].flip = lflip[k];
        }
        for (int i = 0; i < qn; ++i) hr[i] = queue[i];
        be.h2d(mainb[cur], hm.data(), sizeof(CafeMainBucket) * (size_t)n1);
        be.h2d(lrub[cur], hl.data(), sizeof(CafeLruBucket) * (size_t)n2);
        be.h2d(ring, hr.data(), 4 * ((size_t)ring_mask + 1));
        q_head = 0; q_size = qn;
        return be.ok() ? CAFE_OK : CAFE_ERR_CUDA;
    }

private:
    int gate_seg = -1;
    int32_t job_serial = 0;
    bool cursors_advanced = false;
    const uint32_t* presorted_gid = nullptr;
    int presorted_n = 0;
    bool ready = false;
    int cap = 0, cur = 0;
    CafeMainBucket* mainb[2] = {nullptr, nullptr};
    CafeLruBucket* lrub[2] = {nullptr, nullptr};
    uint32_t* ring = nullptr;
    int32_t *ord1 = nullptr, *ord2 = nullptr, *start1 = nullptr, *start2 = nullptr, *beg1 = nullptr, *beg2 = nullptr;
    uint32_t *sgid1 = nullptr, *sgid2 = nullptr;   // ids in the order of ord1 / ord2
    float *simp1 = nullptr, *simp2 = nullptr;      // counts in the order of ord1 / ord2
    CafeEvent* ev = nullptr;
    int32_t* head = nullptr;
    int32_t* nxt = nullptr;
    uint8_t *mark_own = nullptr, *mstate = nullptr, *mark2 = nullptr, *lstate = nullptr, *mflag = nullptr, *lflag = nullptr;
    uint8_t *mark_w1[2] = {nullptr, nullptr}, *mark_c2 = nullptr;   // see CafeJob::mark_in1
    int mark_par = 0;
    int32_t *tl_slot = nullptr, *tl_info = nullptr, *tl_size = nullptr, *tl_rank = nullptr, *tl_grp = nullptr, *tl_head = nullptr;
    int32_t *tl_blk = nullptr, *nmiss = nullptr;
    uint32_t* pushbuf = nullptr;
    CafeFn* tl_agg = nullptr;
    int32_t* ins_res = nullptr;
    CafeRoundResult* res_dev = nullptr;
    size_t off_mark2 = 0, off_res = 0, span_clear = 0;
    CafeSeqState* seq_dev = nullptr;
    uint32_t* cand_key[2] = {nullptr, nullptr};
    int32_t* cand_val[2] = {nullptr, nullptr};
    int32_t* cand_cnt = nullptr;
    int32_t* reset_out = nullptr;

    void release() {
        if (!ready && !mainb[0]) return;
        void* ptrs[] = {mainb[0], mainb[1], lrub[0], lrub[1], ring, sgid1, sgid2, simp1, simp2, ord1, ord2, start1, start2, beg1, beg2, ev, head, nxt, mark_own, mstate, lstate, mark_w1[0], mflag, lflag, tl_slot, tl_info, tl_size, tl_rank, tl_grp, tl_head, pushbuf, tl_blk, tl_agg, nmiss,
                        ins_res, seq_dev, cand_key[0], cand_key[1],
                        cand_val[0], cand_val[1], cand_cnt, reset_out};
        for (void* p : ptrs) if (p) be.free(p);
        mainb[0] = mainb[1] = nullptr; lrub[0] = lrub[1] = nullptr;
        ready = false;
    }

    // prologue of batch_insert / batch_insert_val (sketch.cpp:267-275, 282-291)
    void call_boundary() {
        ++batch_num;
        ++stats.calls;
        decay_importance *= alpha;
        if (decay_importance > CAFE_DECAY_BASE) {
            decay_importance /= CAFE_DECAY_BASE;
            thr = (float)((double)thr / CAFE_DECAY_BASE);
            gflip ^= 1u;
            ++stats.flips;
        }
        if ((double)real_n > lim * 1.2 && adjust) {
            int rc = refit_threshold();
            if (rc == CAFE_ERR_RESET_UNDERFLOW) last_status = rc;   // reported, insert still proceeds
        }
    }

    int run_sequential(const uint32_t* gid, const float* imp, int n, int32_t* mask, int32_t* post_row) {
        CafeSeqState S;
        S.mb = mainb[cur]; S.lb = lrub[cur]; S.ring = ring; S.ring_mask = ring_mask; S.n1 = n1; S.n2 = n2;
        S.thr = thr; S.gflip = gflip; S.real_n = real_n; S.num = num; S.t = t; S.q_head = q_head; S.q_size = q_size;
        S.error = 0;
        be.seq_insert(seq_dev, &S, gid, imp, n, mask);   // runs, then copies the updated scalars back into S
        if (!be.ok()) return last_status = CAFE_ERR_CUDA;
        real_n = S.real_n; num = S.num; t = S.t; q_head = S.q_head; q_size = S.q_size;
        if (S.error) return last_status = CAFE_ERR_CAPACITY;
        if (post_row) be.post_query(mainb[cur], n1, gid, n, mask, post_row);
        return be.ok() ? CAFE_OK : CAFE_ERR_CUDA;
    }

    // Parallel rounds over the segments seg[0..nseg] (positions relative to the sorted stretch of M
    // lookups that gid/imp/mask/post_row point to).  On return *done = number of leading segments
    // committed (fewer than nseg when a threshold re-fit is due at an inner boundary).
    int run_parallel(const uint32_t* gid, const float* imp, int M, const int* seg, int nseg, int32_t* mask,
                     int32_t* post_row, int* done) {
        CafeJob J;
        memset(&J, 0, sizeof(J));
        cursors_advanced = false;
        J.gid = gid; J.imp = imp; J.M = M; J.begin = seg[0]; J.limit = seg[nseg]; J.nseg = nseg;
        for (int i = 0; i <= nseg; ++i) J.seg_off[i] = seg[i];
        for (int i = nseg + 1; i <= CAFE_MAX_SEGMENTS; ++i) J.seg_off[i] = INT32_MAX;
        J.ord1 = ord1; J.start1 = start1; J.beg1 = beg1; J.ord2 = ord2; J.start2 = start2; J.beg2 = beg2;
        J.sgid1 = sgid1; J.sgid2 = sgid2; J.simp1 = imp ? simp1 : nullptr; J.simp2 = imp ? simp2 : nullptr;
        J.n1 = n1; J.n2 = n2; J.thr = thr; J.gflip = gflip; J.t0 = t;
        J.ring = ring; J.ring_mask = ring_mask; J.q_head = q_head; J.q_size = q_size;
        J.main_in = mainb[cur]; J.main_out = mainb[cur ^ 1];
        J.lru_in = lrub[cur]; J.lru_out = lrub[cur ^ 1];
        J.ev = ev; J.head = head; J.nxt = nxt; J.mark_own = mark_own; J.mstate = mstate; J.mark2 = mark2; J.lstate = lstate;
        J.mark_in1 = mark_w1[mark_par]; J.mark_out1 = mark_w1[mark_par ^ 1]; J.mark_c2 = mark_c2;
        J.mflag = mflag; J.lflag = lflag; J.ins_res = ins_res;
        J.tl_slot = tl_slot; J.tl_info = tl_info; J.tl_size = tl_size; J.tl_rank = tl_rank; J.tl_grp = tl_grp; J.tl_head = tl_head;
        J.pushbuf = pushbuf; J.tl_blk = tl_blk; J.tl_agg = tl_agg; J.nmiss = nmiss;
        J.mask = mask;
        J.post_row = post_row;
        J.res = res_dev;
        ++stats.jobs;
        if (++job_serial <= 0) job_serial = 1;
        J.serial = job_serial;
        {
            const size_t span = (size_t)(J.limit - J.begin);
            be.fills(ins_res + J.begin, 0, 4 * span, mflag + J.begin, 0, span,
                     ev + J.begin, 0, sizeof(CafeEvent) * span,   // kind 0 = no event
                     mark2, 0, span_clear - off_mark2);           // mark2 + round result, for the first round
        }

        CafeRoundResult R;
        int rounds = 0;
        bool truncated = false, shortened = false, tl_changed_prev = true;
        int dropped_from = 0, dropped_to = 0;   // positions a shortening has just dropped from the job
        bool first = true;
        for (;;) {
            if (rounds >= round_cap) {
                // state untouched so far (rounds only write the other image): sequential fallback
                ++stats.seq_fallbacks;
                last_status = CAFE_ERR_NOCONVERGE;
                *done = 1;
                const int b0 = J.begin, n0 = J.seg_off[1] - J.begin;
                int rc = run_sequential(gid + b0, imp ? imp + b0 : nullptr, n0, mask + b0, post_row ? post_row + b0 : nullptr);
                return rc == CAFE_OK ? CAFE_OK : rc;
            }
            J.first_round = first ? 1 : 0;
            J.mark_in1 = mark_w1[mark_par]; J.mark_out1 = mark_w1[mark_par ^ 1];
            mark_par ^= 1;   // what this round marks is what the next one reads
            J.all_active = first ? 1 : 0;
            J.cand_active = (first || tl_changed_prev) ? 1 : 0;
            J.final_pass = 0;
            J.lists_stale = shortened ? 1 : 0;
            // a job that has just been shortened: only what the dropped lookups touched replays (marked for this round)
            if (shortened) be.mark_cut(J, dropped_from, dropped_to, const_cast<uint8_t*>(J.mark_in1));
            shortened = false;
            if (!first) {   // (the first round's mark2 + round result were cleared with the job's arrays)
                be.fills(head, 0xff, 4 * (size_t)n1, mark_own, 0, span_clear);   // mark_own + mark2 + round result
                be.route(J);
            }
            be.sort_join(1);
            be.main_pass(J);
            be.sort_join(2);
            be.lru_pass(J);
            be.resolve(J);
            be.d2h(&R, res_dev, sizeof(R));
            if (!be.ok()) return last_status = CAFE_ERR_CUDA;
            ++rounds; ++stats.rounds;
            first = false;
            tl_changed_prev = R.tl_changed != 0;
            if (R.error) return last_status = CAFE_ERR_CAPACITY;
            // A threshold re-fit is due at the first inner boundary where real_n exceeds 1.2*lim.  The
            // per-segment deltas of a round that has not converged yet are estimates, but shrinking
            // the job to an estimated cut is always safe: whatever prefix is kept is iterated to
            // convergence and checked again before it is committed, and the next job starts with the
            // exact boundary test.  Cutting early saves replaying segments that would be discarded.
            if (adjust) {
                int rn = real_n, cut = -1;
                for (int b = 1; b < nseg; ++b) {
                    rn += R.seg_real_delta[b - 1];
                    if ((double)rn > lim * 1.2) { cut = b; break; }
                }
                if (cut > 0) {
                    dropped_from = J.seg_off[cut]; dropped_to = J.limit;
                    J.limit = J.seg_off[cut];
                    J.nseg = cut;
                    nseg = cut;
                    if (!truncated) ++stats.truncated_jobs;
                    truncated = true;
                    shortened = true;   // bucket images written so far may include lookups beyond the new end
                    if (J.limit == J.begin) { *done = cut; return CAFE_OK; }   // empty prefix: nothing to commit
                    continue;
                }
            }
            if (R.changed) continue;
            break;
        }
        // converged: the timeline just produced equals the one consumed
        J.first_round = 0; J.all_active = 0; J.cand_active = 1;
        if (post_row) {
            be.fills(post_row + J.begin, 0, 4 * (size_t)(J.limit - J.begin), head, 0xff, 4 * (size_t)n1, mark_own, 0, (size_t)n1);
            be.route(J);
            J.final_pass = 1;
            be.main_pass(J);
            J.final_pass = 0;
        }
        be.finalize(J);   // per-lookup results, LRU clock values, cursors of the sorted order
        cursors_advanced = true;
        if (R.n_push > 0) be.commit_queue(ring, ring_mask, q_head, q_size, R.n_pop_ok, pushbuf, R.n_push);
        cur ^= 1;
        q_head += (uint32_t)R.n_pop_ok;
        q_size += R.n_push - R.n_pop_ok;
        t += R.n_miss;
        num += R.n_pop_ok;   // every successful pop hands out one hot row (sketch.cpp:176,206,224)
        int grown = 0;
        for (int b = 0; b < nseg; ++b) grown += R.seg_real_delta[b];
        real_n += grown;
        if (J.limit > J.begin) {
            const double r = (double)grown / (J.limit - J.begin);
            cross_rate = cross_rate < 0 ? r : 0.5 * cross_rate + 0.5 * r;
        }
        stats.main_hits += (int64_t)(J.limit - J.begin) - R.n_miss; stats.lru_visits += R.n_miss; stats.events += R.n_events;
        if (rounds > stats.max_rounds) stats.max_rounds = rounds;
        *done = nseg;
        return be.ok() ? CAFE_OK : CAFE_ERR_CUDA;
    }

};
