/*
 * hotsketch_oracle.c -- TEST INFRASTRUCTURE ONLY (never linked or loaded by the product).
 *
 * A sequential, single-threaded CPU restatement, in plain C, of the CAFE+ HotSketch that the
 * reference implements in tricks/sketch.cpp.  It exists so that the CUDA kernels can be compared
 * against the reference's algorithm on identical inputs; only tests, the smoke check and the
 * CPU-baseline leg of the benchmark may call it.
 *
 * Parity status: PINNED.  The reference ships no golden vectors for this path, so the restatement
 * is pinned against (a) the reference itself, compiled from its own source with three mechanical
 * fixes (see build_ref.sh) and driven with the same seeded streams, and (b) the three known-answer
 * hashes stored in tests/golden/kat_hashes.json that the patched reference reproduces.
 *
 * Differences from the reference that are deliberate and documented:
 *   - state is per instance instead of process-global (alpha, decay_importance, batch counter and
 *     global flip bit live in the instance; tricks/sketch.cpp:7-13 keeps them at file scope);
 *   - outputs go to caller buffers instead of the static 16384-entry arrays (sketch.cpp:10);
 *   - ties in reset() are ordered canonically: main table before LRU table, then bucket, then slot
 *     (the reference orders ties by heap address, sketch.cpp:79-96, which varies between runs);
 *   - reset() with fewer candidates than `lim` is refused (returns without change and counts the
 *     event) where the reference would index a vector with a negative number (sketch.cpp:98-112).
 *
 * Each function cites the reference lines it follows.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HS_SLOTS 4
#define HS_DECAY_BASE 10000.0 /* sketch.cpp:8  (V) */

typedef struct {            /* sketch.cpp:23-28 */
    uint32_t val[HS_SLOTS];
    float cnt[HS_SLOTS];
    int32_t dic[HS_SLOTS];
    uint8_t flip;
} hs_main_bucket;

typedef struct {            /* sketch.cpp:29-35 */
    uint32_t val[HS_SLOTS];
    float cnt[HS_SLOTS];
    int32_t dic[HS_SLOTS];
    int32_t t[HS_SLOTS];
    uint8_t flip;
} hs_lru_bucket;

typedef struct hs_oracle {
    int lim, n1, n2;
    int adjust;
    float thr;
    int real_n, num, t;
    double alpha, decay_importance;
    int batch_num;
    uint8_t gflip;
    hs_main_bucket *mb;
    hs_lru_bucket *lb;
    /* FIFO of free hot rows (sketch.cpp:37,55-56) as a ring */
    uint32_t *q;
    int64_t q_cap, q_head, q_size;
    /* event counters (diagnostics only) */
    int64_t n_reset, n_reset_refused, n_flip;
    int64_t n_main_hit, n_lru_hit, n_lru_new, n_promote_own, n_promote_victim, n_insert_fail;
} hs_oracle;

/* ---- FIFO ---------------------------------------------------------------------------------- */
static int q_empty(const hs_oracle *h) { return h->q_size == 0; }
static void q_push(hs_oracle *h, uint32_t id) {
    if (h->q_size >= h->q_cap) abort(); /* cannot happen: ids are conserved */
    h->q[(h->q_head + h->q_size) % h->q_cap] = id;
    h->q_size++;
}
static uint32_t q_pop(hs_oracle *h) {
    uint32_t id = h->q[h->q_head];
    h->q_head = (h->q_head + 1) % h->q_cap;
    h->q_size--;
    return id;
}

/* ---- hashing: sketch.cpp:38-43 ------------------------------------------------------------- */
static int hash_main(const hs_oracle *h, uint32_t x) { return (int)((int64_t)x * 1000000007LL % h->n1); }
static int hash_lru(const hs_oracle *h, uint32_t x) { return (int)((int64_t)x * 1000000007LL % h->n2); }

/* ---- lazy decay by flip bit: sketch.cpp:130-140 -------------------------------------------- */
static void touch_main(hs_oracle *h, hs_main_bucket *b) {
    if (b->flip != h->gflip) {
        b->flip = h->gflip;
        for (int i = 0; i < HS_SLOTS; ++i) b->cnt[i] = (float)((double)b->cnt[i] / HS_DECAY_BASE);
    }
}
static void touch_lru(hs_oracle *h, hs_lru_bucket *b) {
    if (b->flip != h->gflip) {
        b->flip = h->gflip;
        for (int i = 0; i < HS_SLOTS; ++i) b->cnt[i] = (float)((double)b->cnt[i] / HS_DECAY_BASE);
    }
}

/* ---- construction: sketch.cpp:44-70, 309-313 ----------------------------------------------- */
hs_oracle *hs_new(int lim, float thr, int adjust, double alpha) {
    hs_oracle *h = (hs_oracle *)calloc(1, sizeof(hs_oracle));
    h->lim = lim;
    h->thr = thr;
    h->adjust = adjust;
    h->alpha = alpha;
    h->decay_importance = 1.0;
    h->n1 = (int)(lim * 0.9);
    h->n2 = (int)(lim * 0.1);
    h->mb = (hs_main_bucket *)calloc((size_t)(h->n1 > 0 ? h->n1 : 1), sizeof(hs_main_bucket));
    h->lb = (hs_lru_bucket *)calloc((size_t)(h->n2 > 0 ? h->n2 : 1), sizeof(hs_lru_bucket));
    h->q_cap = (int64_t)lim + 8;
    h->q = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)h->q_cap);
    for (int i = 1; i < lim; ++i) q_push(h, (uint32_t)i);
    return h;
}

void hs_free(hs_oracle *h) {
    if (!h) return;
    free(h->mb);
    free(h->lb);
    free(h->q);
    free(h);
}

/* ---- query: sketch.cpp:118-128 ------------------------------------------------------------- */
static int32_t query_one(const hs_oracle *h, uint32_t x) {
    const hs_main_bucket *b = &h->mb[hash_main(h, x)];
    for (int i = 0; i < HS_SLOTS; ++i)
        if (b->val[i] == x && b->dic[i]) return -b->dic[i];
    return (int32_t)x;
}

/* ---- presence probe used by analyse1: sketch.cpp:142-150 ----------------------------------- */
static int present_one(const hs_oracle *h, uint32_t x) {
    const hs_main_bucket *b = &h->mb[hash_main(h, x)];
    for (int i = 0; i < HS_SLOTS; ++i)
        if (b->val[i] == x) return 1;
    return 0;
}

/* ---- Insert into the main table (promotion target): sketch.cpp:232-259 --------------------- */
static int promote_into_main(hs_oracle *h, uint32_t x, float count, int32_t carried) {
    hs_main_bucket *b = &h->mb[hash_main(h, x)];
    int min_i = -1;
    float min_cnt = 1e9f;
    touch_main(h, b);
    for (int i = 0; i < HS_SLOTS; ++i) {
        if (b->val[i] == 0) {
            b->val[i] = x;
            b->cnt[i] = count;
            b->dic[i] = carried;
            return 1;
        }
        if (b->cnt[i] < min_cnt) {
            min_cnt = b->cnt[i];
            min_i = i;
        }
    }
    if (min_i < 0) { /* every cnt >= 1e9: the reference would index slot -1 */
        if (carried != 0) q_push(h, (uint32_t)carried);
        h->n_insert_fail++;
        return 0;
    }
    if (!b->dic[min_i]) {
        b->cnt[min_i] += count;
        b->val[min_i] = x;
        b->dic[min_i] = carried;
        return 1;
    }
    if (carried != 0) q_push(h, (uint32_t)carried);
    h->n_insert_fail++;
    return 0;
}

/* ---- LRU filter stage: sketch.cpp:161-210 --------------------------------------------------- */
static int insert_lru(hs_oracle *h, uint32_t x, float count) {
    hs_lru_bucket *b = &h->lb[hash_lru(h, x)];
    int p = -1, t_min = 1000000000, got = 0;
    touch_lru(h, b);
    for (int i = 0; i < HS_SLOTS; ++i) {
        if (b->val[i] == x) {
            h->n_lru_hit++;
            b->t[i] = ++h->t;
            b->cnt[i] += count;
            if (b->cnt[i] >= h->thr && b->cnt[i] - count < h->thr) h->real_n++;
            if (b->cnt[i] >= h->thr && !q_empty(h) && !b->dic[i]) {
                b->dic[i] = (int32_t)q_pop(h);
                got = 1;
                h->num++;
            }
            if (b->cnt[i] >= h->thr) {
                h->n_promote_own++;
                if (!promote_into_main(h, b->val[i], b->cnt[i], b->dic[i])) got = 0;
                b->val[i] = 0;
                b->t[i] = 0;
                b->cnt[i] = 0;
                b->dic[i] = 0;
            }
            return got;
        }
        if (t_min > b->t[i]) {
            t_min = b->t[i];
            p = i;
        }
    }
    if (b->dic[p] || b->cnt[p] >= 5) {
        h->n_promote_victim++;
        promote_into_main(h, b->val[p], b->cnt[p], b->dic[p]);
    }
    h->n_lru_new++;
    b->val[p] = x;
    b->t[p] = ++h->t;
    b->cnt[p] = 1;
    b->dic[p] = 0;
    if (b->cnt[p] >= h->thr && b->cnt[p] - count < h->thr) h->real_n++;
    if (b->cnt[p] >= h->thr && !q_empty(h) && !b->dic[p]) {
        b->dic[p] = (int32_t)q_pop(h);
        got = 1;
        h->num++;
    }
    return got;
}

/* ---- one lookup: sketch.cpp:211-231 --------------------------------------------------------- */
static int insert_one(hs_oracle *h, uint32_t x, float count) {
    hs_main_bucket *b = &h->mb[hash_main(h, x)];
    int got = 0;
    touch_main(h, b);
    for (int i = 0; i < HS_SLOTS; ++i) {
        if (b->val[i] == x) {
            h->n_main_hit++;
            b->cnt[i] += count;
            float c = b->cnt[i];
            if (c >= h->thr && c - count < h->thr) h->real_n++;
            if (c >= h->thr && !b->dic[i] && !q_empty(h)) {
                b->dic[i] = (int32_t)q_pop(h);
                got = 1;
                h->num++;
            }
            return got;
        }
    }
    return insert_lru(h, x, count);
}

/* ---- adaptive threshold: sketch.cpp:76-116 -------------------------------------------------- */
typedef struct {
    float cnt;
    int32_t order; /* canonical position: main slots first, then LRU slots */
} hs_cand;

static int cand_less(const void *a, const void *b) {
    const hs_cand *x = (const hs_cand *)a, *y = (const hs_cand *)b;
    if (x->cnt < y->cnt) return -1;
    if (x->cnt > y->cnt) return 1;
    return (x->order > y->order) - (x->order < y->order);
}

static int32_t *slot_dic(hs_oracle *h, int32_t order) {
    int32_t main_slots = h->n1 * HS_SLOTS;
    if (order < main_slots) return &h->mb[order / HS_SLOTS].dic[order % HS_SLOTS];
    order -= main_slots;
    return &h->lb[order / HS_SLOTS].dic[order % HS_SLOTS];
}

void hs_reset(hs_oracle *h) {
    size_t cap = (size_t)(h->n1 + h->n2) * HS_SLOTS;
    hs_cand *vec = (hs_cand *)malloc(sizeof(hs_cand) * (cap ? cap : 1));
    int l = 0;
    for (int k = 0; k < h->n1; ++k) {
        touch_main(h, &h->mb[k]);
        for (int i = 0; i < HS_SLOTS; ++i)
            if (h->mb[k].cnt[i] >= h->thr || h->mb[k].dic[i]) {
                vec[l].cnt = h->mb[k].cnt[i];
                vec[l].order = k * HS_SLOTS + i;
                ++l;
            }
    }
    for (int k = 0; k < h->n2; ++k) {
        touch_lru(h, &h->lb[k]);
        for (int i = 0; i < HS_SLOTS; ++i)
            if (h->lb[k].cnt[i] >= h->thr || h->lb[k].dic[i]) {
                vec[l].cnt = h->lb[k].cnt[i];
                vec[l].order = h->n1 * HS_SLOTS + k * HS_SLOTS + i;
                ++l;
            }
    }
    if (l < h->lim) { /* reference: negative vector index (undefined); refuse instead */
        h->n_reset_refused++;
        free(vec);
        return;
    }
    qsort(vec, (size_t)l, sizeof(hs_cand), cand_less);
    for (int i = 0; i <= l - h->lim; ++i) {
        int32_t *d = slot_dic(h, vec[i].order);
        if (*d != 0) {
            q_push(h, (uint32_t)*d);
            *d = 0;
        }
    }
    for (int i = l - h->lim + 1; i < l; ++i) {
        int32_t *d = slot_dic(h, vec[i].order);
        if (*d == 0 && !q_empty(h)) *d = (int32_t)q_pop(h);
    }
    h->thr = vec[l - h->lim].cnt;
    h->real_n = h->lim;
    h->n_reset++;
    free(vec);
}

/* ---- per-call prologue shared by batch_insert / batch_insert_val: sketch.cpp:267-275,282-291 - */
static void call_boundary(hs_oracle *h) {
    h->batch_num++;
    h->decay_importance *= h->alpha;
    if (h->decay_importance > HS_DECAY_BASE) {
        h->decay_importance /= HS_DECAY_BASE;
        h->thr = (float)((double)h->thr / HS_DECAY_BASE);
        h->gflip ^= 1;
        h->n_flip++;
    }
    if ((double)h->real_n > h->lim * 1.2 && h->adjust) hs_reset(h);
}

/* ---- batch entry points: sketch.cpp:260-296 ------------------------------------------------- */
void hs_batch_query(const hs_oracle *h, const uint32_t *ids, int n, int32_t *out) {
    for (int i = 0; i < n; ++i) out[i] = query_one(h, ids[i]);
}

/* v == NULL gives the unit-count variant (batch_insert, sketch.cpp:266-280). */
void hs_batch_insert_val(hs_oracle *h, const uint32_t *ids, const float *v, int n, int32_t *out) {
    call_boundary(h);
    for (int i = 0; i < n; ++i) out[i] = insert_one(h, ids[i], v ? v[i] : 1.0f);
}

/* ---- diagnostics: sketch.cpp:314-327 -------------------------------------------------------- */
double hs_analyse(const hs_oracle *h, const uint32_t *ids, int n) {
    int a = 0;
    for (int i = 0; i < n; ++i) a += query_one(h, ids[i]) < 0;
    return 1.0 * a / n;
}
double hs_analyse1(const hs_oracle *h, const uint32_t *ids, int n) {
    int a = 0;
    for (int i = 0; i < n; ++i) a += present_one(h, ids[i]);
    return 1.0 * a / n;
}

/* ---- state export for bit-exact comparison --------------------------------------------------- */
int hs_n1(const hs_oracle *h) { return h->n1; }
int hs_n2(const hs_oracle *h) { return h->n2; }

/* scalars[0..7] = thr(bits), real_n, num, t, gflip, q_size, batch_num, n_reset */
void hs_scalars(const hs_oracle *h, int64_t *out, double *decay_importance) {
    uint32_t bits;
    memcpy(&bits, &h->thr, 4);
    out[0] = bits;
    out[1] = h->real_n;
    out[2] = h->num;
    out[3] = h->t;
    out[4] = h->gflip;
    out[5] = h->q_size;
    out[6] = h->batch_num;
    out[7] = h->n_reset;
    if (decay_importance) *decay_importance = h->decay_importance;
}

/* counters[0..8] = main_hit, lru_hit, lru_new, promote_own, promote_victim, insert_fail, resets,
 * resets_refused, flips */
void hs_counters(const hs_oracle *h, int64_t *out) {
    out[0] = h->n_main_hit;
    out[1] = h->n_lru_hit;
    out[2] = h->n_lru_new;
    out[3] = h->n_promote_own;
    out[4] = h->n_promote_victim;
    out[5] = h->n_insert_fail;
    out[6] = h->n_reset;
    out[7] = h->n_reset_refused;
    out[8] = h->n_flip;
}

/* Arrays are [n1*4] / [n2*4], bucket-major; flip arrays are [n1] / [n2]. */
void hs_dump_main(const hs_oracle *h, uint32_t *val, float *cnt, int32_t *dic, uint8_t *flip) {
    for (int k = 0; k < h->n1; ++k) {
        for (int i = 0; i < HS_SLOTS; ++i) {
            val[k * HS_SLOTS + i] = h->mb[k].val[i];
            cnt[k * HS_SLOTS + i] = h->mb[k].cnt[i];
            dic[k * HS_SLOTS + i] = h->mb[k].dic[i];
        }
        flip[k] = h->mb[k].flip;
    }
}
void hs_dump_lru(const hs_oracle *h, uint32_t *val, float *cnt, int32_t *dic, int32_t *t, uint8_t *flip) {
    for (int k = 0; k < h->n2; ++k) {
        for (int i = 0; i < HS_SLOTS; ++i) {
            val[k * HS_SLOTS + i] = h->lb[k].val[i];
            cnt[k * HS_SLOTS + i] = h->lb[k].cnt[i];
            dic[k * HS_SLOTS + i] = h->lb[k].dic[i];
            t[k * HS_SLOTS + i] = h->lb[k].t[i];
        }
        flip[k] = h->lb[k].flip;
    }
}
/* Writes the queue front-to-back; returns its length (out may be NULL to ask for the length). */
int64_t hs_dump_queue(const hs_oracle *h, uint32_t *out) {
    if (out)
        for (int64_t i = 0; i < h->q_size; ++i) out[i] = h->q[(h->q_head + i) % h->q_cap];
    return h->q_size;
}
