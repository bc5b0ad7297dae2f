/*
 * sigmod_oracle.c -- TEST INFRASTRUCTURE ONLY (never linked or loaded by the product).
 *
 * A sequential CPU restatement, in plain C, of the one-stage HotSketch of the reference's artifact tree
 * (ArtifactEvaluation/embeddings/sketch.cpp, class SS: the sketch of the SIGMOD'24 CAFE paper): `lim`
 * buckets of four slots kept sorted by count, Space-Saving replacement of the last slot, a FIFO of free
 * hot rows, and a multiplicative decay of all counts once the inserted mass exceeds 10 * lim * k.
 *
 * Parity status: PINNED against the reference itself, compiled from its own source by build_ref.sh
 * (oracle/_ref/libsketch_sigmod_ref.so) and driven with the same seeded streams (tests/test_oracle_sigmod.py),
 * and against tests/golden/sigmod_stream.npz, which that library produced.
 *
 * Deliberate differences: state is per instance (the reference keeps ss[26] at file scope, :151); outputs go
 * to caller buffers instead of the static 16384-entry arrays (:7).  Slot values of never-used slots are zero
 * here and uninitialised in the reference (:38-41 clear cnt and dic only); they are never compared while the
 * slot's count is zero, so no result depends on them.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct { uint32_t val[4]; float cnt[4]; int32_t dic[4]; } sg_bucket;   /* sketch.cpp:17-21 */

typedef struct {
    int k, s, lim, num;          /* :11-12  (Threshold = k, s = lim) */
    double tot, decay_rate;      /* :13-15 */
    sg_bucket* b;
    uint32_t* q;                 /* FIFO of free hot rows (:26) as a ring */
    int64_t q_cap, q_head, q_size;
    int64_t decays;
} sg_oracle;

static void q_push(sg_oracle* o, uint32_t id) { o->q[(o->q_head + o->q_size) % o->q_cap] = id; o->q_size++; }
static uint32_t q_pop(sg_oracle* o) { uint32_t id = o->q[o->q_head % o->q_cap]; o->q_head++; o->q_size--; return id; }

/* SS::SS, sketch.cpp:28-42 */
sg_oracle* sg_new(int k, int lim, double dr) {
    sg_oracle* o = (sg_oracle*)calloc(1, sizeof(sg_oracle));
    o->k = k; o->lim = lim; o->s = lim; o->decay_rate = dr; o->tot = 0; o->num = 0;
    o->b = (sg_bucket*)calloc((size_t)lim, sizeof(sg_bucket));
    o->q_cap = (int64_t)lim + 8;
    o->q = (uint32_t*)calloc((size_t)o->q_cap, sizeof(uint32_t));
    for (int i = 1; i < lim; ++i) q_push(o, (uint32_t)i);
    return o;
}
void sg_free(sg_oracle* o) { if (o) { free(o->b); free(o->q); free(o); } }

static uint32_t sg_hash(const sg_oracle* o, uint32_t val) { return val % (uint32_t)o->s; }   /* :22-24 */

/* SS::query, :43-51 */
static int32_t sg_query1(const sg_oracle* o, uint32_t val) {
    const sg_bucket* b = &o->b[sg_hash(o, val)];
    for (int i = 0; i < 4; ++i)
        if (b->cnt[i] != 0 && b->val[i] == val) { if (b->dic[i]) return -b->dic[i]; }
    return (int32_t)val;
}
void sg_batch_query(sg_oracle* o, const uint32_t* data, int len, int32_t* out) {
    for (int i = 0; i < len; ++i) out[i] = sg_query1(o, data[i]);
}

/* SS::decay, :76-88 */
static void sg_decay(sg_oracle* o) {
    for (int key = 0; key < o->s; ++key) {
        sg_bucket* b = &o->b[key];
        for (int i = 0; i < 4; ++i) {
            if (b->dic[i] && (double)b->cnt[i] * o->decay_rate < (double)o->k) { q_push(o, (uint32_t)b->dic[i]); b->dic[i] = 0; }
            b->cnt[i] = (float)((double)b->cnt[i] * o->decay_rate);
        }
    }
    o->tot = 0;
    o->decays++;
}

/* SS::Insert, :89-123 */
static int sg_insert1(sg_oracle* o, uint32_t val, float v) {
    o->tot += v;
    sg_bucket* b = &o->b[sg_hash(o, val)];
    int id = 0;
    for (int i = 0; i < 4; ++i) {
        if (b->cnt[i] != 0 && b->val[i] == val) {
            b->cnt[i] += v;
            if (b->cnt[i] >= (float)o->k && o->q_size > 0 && !b->dic[i]) { b->dic[i] = (int32_t)q_pop(o); id = 1; ++o->num; }
            while (i && b->cnt[i] > b->cnt[i - 1]) {
                float c = b->cnt[i]; b->cnt[i] = b->cnt[i - 1]; b->cnt[i - 1] = c;
                uint32_t x = b->val[i]; b->val[i] = b->val[i - 1]; b->val[i - 1] = x;
                int32_t d = b->dic[i]; b->dic[i] = b->dic[i - 1]; b->dic[i - 1] = d;
                --i;
            }
            return id;
        }
    }
    for (int i = 0; i < 4; ++i)
        if (b->cnt[i] == 0) { b->cnt[i] = v; b->val[i] = val; return 0; }
    if (!b->dic[3]) { b->cnt[3] += v; b->val[3] = val; }
    return 0;
}
/* SS::batch_insert_val / batch_insert, :131-149 (v == NULL: unit counts) */
void sg_batch_insert_val(sg_oracle* o, const uint32_t* data, const float* v, int len, int32_t* out) {
    if (o->tot > (double)(1ll * o->s * o->k * 10)) sg_decay(o);
    for (int i = 0; i < len; ++i) out[i] = sg_insert1(o, data[i], v ? v[i] : 1.0f);
}

/* SS::update, :61-75: rebuild the FIFO from the rows the buckets hold (after loading a checkpoint) */
void sg_update(sg_oracle* o) {
    uint8_t* used = (uint8_t*)calloc((size_t)o->lim + 1, 1);
    for (int key = 0; key < o->s; ++key)
        for (int i = 0; i < 4; ++i)
            if (o->b[key].dic[i] > 0 && o->b[key].dic[i] < o->lim) used[o->b[key].dic[i]] = 1;
    o->q_head = 0; o->q_size = 0;
    for (int i = 1; i < o->lim; ++i) if (!used[i]) q_push(o, (uint32_t)i);
    free(used);
}

/* state export: scalars[0..4] = num, queue length, decays, k, lim; tot separately */
void sg_scalars(const sg_oracle* o, int64_t* out, double* tot) {
    out[0] = o->num; out[1] = o->q_size; out[2] = o->decays; out[3] = o->k; out[4] = o->lim;
    if (tot) *tot = o->tot;
}
void sg_dump(const sg_oracle* o, uint32_t* val, float* cnt, int32_t* dic, uint32_t* queue) {
    for (int key = 0; key < o->s; ++key)
        for (int i = 0; i < 4; ++i) {
            /* a slot's id is meaningful only while its count is non-zero */
            val[key * 4 + i] = o->b[key].cnt[i] != 0 ? o->b[key].val[i] : 0;
            cnt[key * 4 + i] = o->b[key].cnt[i];
            dic[key * 4 + i] = o->b[key].dic[i];
        }
    for (int64_t i = 0; i < o->q_size; ++i) queue[i] = o->q[(o->q_head + i) % o->q_cap];
}
