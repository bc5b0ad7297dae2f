// hostemu.cpp -- TEST INFRASTRUCTURE ONLY: a CPU backend for SketchEngine.
//
// It runs the very same per-bucket and per-position functions the CUDA kernels call
// (cafe_b200/csrc/sketch_core.cuh) in plain loops, under the same host-side driver
// (sketch_engine.h), so that the parallel-insert algorithm, the call-boundary logic and the
// threshold re-fit can be compared with the sequential oracle in a container without a GPU.
// Nothing in the product loads this library.
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <numeric>
#include <vector>

#include "../../cafe_b200/csrc/sketch_engine.h"

struct HostBackend {
    // bucket visiting order of the emulated "grid": reversed on odd rounds to show that results do
    // not depend on the order in which threads run
    int flip_order = 0;
    void* alloc(size_t n) { return calloc(n ? n : 1, 1); }
    void free(void* p) { ::free(p); }
    void memset(void* p, int v, size_t n) { ::memset(p, v, n); }
    void fills(void* p0, int v0, size_t n0, void* p1 = nullptr, int v1 = 0, size_t n1 = 0, void* p2 = nullptr, int v2 = 0,
               size_t n2 = 0, void* p3 = nullptr, int v3 = 0, size_t n3 = 0) {
        if (p0 && n0) ::memset(p0, v0, n0);
        if (p1 && n1) ::memset(p1, v1, n1);
        if (p2 && n2) ::memset(p2, v2, n2);
        if (p3 && n3) ::memset(p3, v3, n3);
    }
    void fill_iota(uint32_t* p, int n, uint32_t first) { for (int i = 0; i < n; ++i) p[i] = first + (uint32_t)i; }
    void h2d(void* d, const void* s, size_t n) { memcpy(d, s, n); }
    void copy(void* d, const void* s, size_t n) { memcpy(d, s, n); }
    void advance_cursors(const int32_t* ord, const int32_t* start, int32_t* beg, int nb, int limit) {
        for (int k = 0; k < nb; ++k) beg[k] = cafe_advance_cursor(ord, beg[k], start[k + 1], limit);
    }
    void d2h(void* d, const void* s, size_t n) { memcpy(d, s, n); }
    bool ok() { return true; }
    bool prepare(int, int, int) { return true; }

    void query(const CafeMainBucket* mb, int n1, const uint32_t* gid, int n, int32_t* out) {
        for (int i = 0; i < n; ++i) {
            int32_t r = cafe_probe_hot(mb[cafe_hash(gid[i], n1)], gid[i]);
            out[i] = r ? -r : (int32_t)gid[i];
        }
    }
    void post_query(const CafeMainBucket* mb, int n1, const uint32_t* gid, int n, const int32_t* mask, int32_t* out) {
        for (int i = 0; i < n; ++i) out[i] = mask[i] ? cafe_probe_hot(mb[cafe_hash(gid[i], n1)], gid[i]) : 0;
    }
    void sort_join(int) {}
    void wait_gate() {}
    void sort_lookups(const uint32_t* gid, int M, int nb, int32_t* ord, uint32_t* sgid, int32_t* start, int32_t* beg, int lane) {
        (void)lane;
        sort_lookups_impl(gid, M, nb, ord, start);
        for (int i = 0; i < M; ++i) sgid[i] = gid[ord[i]];
        memcpy(beg, start, 4 * (size_t)nb);
    }
    void gather_counts(const float* imp, const int32_t* ord1, const int32_t* ord2, int M, float* simp1, float* simp2) {
        for (int i = 0; i < M; ++i) { simp1[i] = imp[ord1[i]]; simp2[i] = imp[ord2[i]]; }
    }
    void sort_lookups_impl(const uint32_t* gid, int M, int nb, int32_t* ord, int32_t* start) {
        std::vector<int32_t> key((size_t)M);
        for (int i = 0; i < M; ++i) key[i] = cafe_hash(gid[i], nb);
        std::iota(ord, ord + M, 0);
        std::stable_sort(ord, ord + M, [&](int32_t a, int32_t b) { return key[a] < key[b]; });
        int j = 0;
        for (int k = 0; k <= nb; ++k) {
            while (j < M && key[ord[j]] < k) ++j;
            start[k] = j;
        }
    }
    void main_pass(const CafeJob& J) {
        flip_order ^= 1;
        if (flip_order) for (int k = J.n1 - 1; k >= 0; --k) cafe_main_pass_bucket(J, k);
        else for (int k = 0; k < J.n1; ++k) cafe_main_pass_bucket(J, k);
    }
    void mark_cut(const CafeJob& J, int from, int to, uint8_t* mark_next1) {
        for (int p = from; p < to; ++p) cafe_mark_cut_position(J, p, mark_next1);
    }
    void route(const CafeJob& J) {
        for (int p = J.limit - 1; p >= J.begin; --p) cafe_route_position(J, p);
    }
    // per-lookup results and the LRU clock numbering, once the rounds have converged
    void finalize(const CafeJob& J) {
        int32_t misses = 0;
        for (int p = J.begin; p < J.limit; ++p) {
            cafe_finalize_position(J, p);
            misses += (J.mflag[p] & CAFE_F_MISS) ? 1 : 0;
            J.nmiss[p] = misses;
        }
        for (int k = 0; k < J.n2; ++k) cafe_lru_tconvert(J, k);
        advance_cursors(J.ord1, J.start1, const_cast<int32_t*>(J.beg1), J.n1, J.limit);
        advance_cursors(J.ord2, J.start2, const_cast<int32_t*>(J.beg2), J.n2, J.limit);
    }
    void lru_pass(const CafeJob& J) {
        if (flip_order) for (int k = J.n2 - 1; k >= 0; --k) cafe_lru_pass_bucket(J, k);
        else for (int k = 0; k < J.n2; ++k) cafe_lru_pass_bucket(J, k);
    }
    void resolve(const CafeJob& J) {
        // list the ops in slot order, updating the previous round's list in place
        const int32_t n_old = J.tl_head[0];
        int32_t j = 0;
        for (int p = J.begin; p < J.limit; ++p) {
            if ((p - J.begin) % CAFE_TL_GROUP == 0) J.tl_grp[(p - J.begin) / CAFE_TL_GROUP] = j;
            const CafeOps o = cafe_ops_of(J, p);
            cafe_tl_emit(J, p, o, j, n_old);
            j += cafe_ops_count(o);
        }
        J.tl_grp[(J.limit - J.begin + CAFE_TL_GROUP - 1) / CAFE_TL_GROUP] = j;
        cafe_tl_set_count(J, j, n_old);
        CafeFn before = cafe_fn_identity();
        for (int32_t i = 0; i < j; ++i) {
            cafe_tl_finish_op(J, i, j, before);
            before = cafe_fn_then(before, cafe_fn_of_info(J.tl_info[i]));
        }
        for (int p = J.begin; p < J.limit; ++p) {
            int c, m;
            cafe_position_counts(J, p, &c, &m);
            if (c) J.res->seg_real_delta[cafe_segment_of(J, p)] += c;
            J.res->n_miss += m;
        }
    }
    void commit_queue(uint32_t* ring, uint32_t mask, uint32_t q_head, int32_t q_size, int32_t n_pop_ok,
                      const uint32_t* pushbuf, int n_push) {
        for (int j = 0; j < n_push; ++j) cafe_commit_push(ring, mask, q_head, q_size, n_pop_ok, pushbuf, j);
    }
    void seq_insert(CafeSeqState* dev, CafeSeqState* S, const uint32_t* gid, const float* imp, int n, int32_t* mask) {
        (void)dev;
        for (int i = 0; i < n; ++i) mask[i] = cafe_seq_insert(*S, gid[i], imp ? imp[i] : 1.0f);
    }
    void reset_collect(CafeMainBucket* mb, CafeLruBucket* lb, int n1, int n2, uint32_t gflip, float thr, int32_t* cnt,
                       uint32_t* key, int32_t* val, int32_t* l_out) {
        (void)cnt;
        int l = 0;
        for (int k = 0; k < n1; ++k) {
            cafe_reset_touch_count_main(mb[k], gflip, thr);
            for (int i = 0; i < 4; ++i)
                if (mb[k].cnt[i] >= thr || mb[k].dic[i] != 0) { key[l] = cafe_float_bits(mb[k].cnt[i]); val[l] = k * 4 + i; ++l; }
        }
        for (int k = 0; k < n2; ++k) {
            cafe_reset_touch_count_lru(lb[k], gflip, thr);
            for (int i = 0; i < 4; ++i)
                if (lb[k].cnt[i] >= thr || lb[k].dic[i] != 0) { key[l] = cafe_float_bits(lb[k].cnt[i]); val[l] = n1 * 4 + k * 4 + i; ++l; }
        }
        *l_out = l;
    }
    void sort_pairs(const uint32_t* kin, const int32_t* vin, uint32_t* kout, int32_t* vout, int n, int bits) {
        (void)bits;
        std::vector<int32_t> idx((size_t)n);
        std::iota(idx.begin(), idx.end(), 0);
        std::stable_sort(idx.begin(), idx.end(), [&](int32_t a, int32_t b) { return kin[a] < kin[b]; });
        for (int i = 0; i < n; ++i) { kout[i] = kin[idx[i]]; vout[i] = vin[idx[i]]; }
    }
    // sketch.cpp:98-115 on the sorted candidates
    void reset_apply(const uint32_t* key, const int32_t* val, int l, int lim, CafeMainBucket* mb, CafeLruBucket* lb,
                     int n1, uint32_t* ring, uint32_t mask, uint32_t q_head, int32_t q_size, int32_t* dev_out,
                     int32_t* out) {
        (void)dev_out;
        int npush = 0, npop = 0;
        const int z = l - lim;
        for (int i = 0; i <= z; ++i) {
            int32_t* d = cafe_slot_dic(mb, lb, n1, val[i]);
            if (*d != 0) { ring[(q_head + (uint32_t)(q_size + npush)) & mask] = (uint32_t)*d; ++npush; *d = 0; }
        }
        const int avail = q_size + npush;
        for (int i = z + 1; i < l; ++i) {
            int32_t* d = cafe_slot_dic(mb, lb, n1, val[i]);
            if (*d == 0 && npop < avail) { *d = (int32_t)ring[(q_head + (uint32_t)npop) & mask]; ++npop; }
        }
        out[0] = (int32_t)key[z];
        out[1] = npush;
        out[2] = npop;
    }
};

typedef SketchEngine<HostBackend> Engine;

extern "C" {
void* emu_new(int lim, float thr, int adjust, double alpha, int cap) {
    Engine* e = new Engine();
    if (e->init(lim, thr, adjust, alpha, cap) != CAFE_OK) { delete e; return nullptr; }
    return e;
}
void emu_free(void* h) { delete (Engine*)h; }
int emu_n1(void* h) { return ((Engine*)h)->n1; }
int emu_n2(void* h) { return ((Engine*)h)->n2; }
int emu_query(void* h, const uint32_t* gid, int n, int32_t* out) { return ((Engine*)h)->query(gid, n, out); }
int emu_insert(void* h, const uint32_t* gid, const float* imp, const int* seg_off, int nseg, int32_t* mask,
               int32_t* post_row, int parallel) {
    return ((Engine*)h)->insert_segments(gid, imp, seg_off, nseg, mask, post_row, parallel != 0);
}
int emu_refit(void* h) { return ((Engine*)h)->refit_threshold(); }
void emu_set_window(void* h, int w) { ((Engine*)h)->window = w; }
void emu_set_round_cap(void* h, int c) { ((Engine*)h)->round_cap = c; }
void emu_set_job_sizing(void* h, int by_rate) { ((Engine*)h)->size_jobs_by_rate = by_rate != 0; }
// scalars[0..7] = thr bits, real_n, num, t, gflip, q_size, batch_num, window
void emu_scalars(void* h, int64_t* out, double* decay) {
    Engine* e = (Engine*)h;
    uint32_t bits;
    memcpy(&bits, &e->thr, 4);
    out[0] = bits; out[1] = e->real_n; out[2] = e->num; out[3] = e->t; out[4] = e->gflip; out[5] = e->q_size;
    out[6] = e->batch_num; out[7] = e->window;
    if (decay) *decay = e->decay_importance;
}
void emu_stats(void* h, int64_t* out) { memcpy(out, &((Engine*)h)->stats, sizeof(CafeSketchStats)); }
void emu_dump(void* h, uint32_t* mval, float* mcnt, int32_t* mdic, uint8_t* mflip, uint32_t* lval, float* lcnt,
              int32_t* ldic, int32_t* lt, uint8_t* lflip, uint32_t* queue) {
    ((Engine*)h)->dump(mval, mcnt, mdic, mflip, lval, lcnt, ldic, lt, lflip, queue);
}
}
