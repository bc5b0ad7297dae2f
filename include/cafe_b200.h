/*
 * cafe_b200.h -- C ABI of libcafe_b200.so: the CAFE compressed-embedding hot path on one B200.
 *
 * Plain C signatures: device and host pointers, sizes, a stream passed as void* (a cudaStream_t; 0 is
 * the default stream).  Every function returns a status (CAFE_OK = 0) unless noted; after
 * CAFE_ERR_CUDA, cafe_last_error() describes the failing call.  A handle belongs to the CUDA device
 * that was current when it was created and must be used by one host thread at a time.
 *
 * Citations give the reference interface each entry point stands in for (paths inside the
 * reference project).
 */
#ifndef CAFE_B200_H
#define CAFE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CAFE_STATUS_ENUMS
#define CAFE_STATUS_ENUMS
enum {
    CAFE_OK = 0,
    CAFE_ERR_ARG = 1,
    CAFE_ERR_CAPACITY = 2,
    CAFE_ERR_CUDA = 3,
    CAFE_ERR_NOCONVERGE = 4,        /* informational: the sequential kernel finished the job; results are exact */
    CAFE_ERR_RESET_UNDERFLOW = 5,   /* informational: a threshold re-fit was refused (fewer candidates than rows) */
    CAFE_ERR_UNSUPPORTED = 6
};
enum { CAFE_INSERT_PARALLEL = 0, CAFE_INSERT_SEQUENTIAL = 1 };
#endif
#define CAFE_MAX_FIELDS 64

const char* cafe_last_error(void);

/* ---- HotSketch, device ABI -------------------------------------------------------------------- */

/* Replaces init(n, Threshold, adjust_thres, alp) (tricks/sketch.cpp:309-313) and the SS constructor
 * (:44-70).  hotn = number of hot rows (`lim`); max_lookups = the largest number of ids any later
 * call will pass (all fields of one fused call together).  All device memory is allocated here. */
int cafe_sketch_create(void** handle, int hotn, float threshold, int adjust_thres, double alpha, int max_lookups);
int cafe_sketch_destroy(void* handle);

/* Replaces batch_query (tricks/sketch.cpp:260-265, 300-302): out[i] = -hot_row if gid[i] is hot, else
 * (int32)gid[i].  Device pointers; no host synchronisation. */
int cafe_sketch_query(void* handle, const uint32_t* gid_dev, int n, int32_t* out_dev, void* stream);

/* Replaces batch_insert_val / batch_insert (tricks/sketch.cpp:266-296, 303-308): nseg consecutive calls,
 * call s covering lookups [seg_off_host[s], seg_off_host[s+1]).  imp_dev == NULL gives batch_insert
 * (unit counts).  mask_dev[i] = the reference's per-lookup result (1 = handed a hot row).
 * post_row_dev (optional) = for lookups with mask 1, the hot row a batch_query right after that
 * lookup's own call would return (0 if none) -- what the module's guarded migration needs.
 * mode: CAFE_INSERT_PARALLEL (round-based, all buckets at once) or CAFE_INSERT_SEQUENTIAL (one
 * thread, the on-device golden path).  Both leave the state the reference's loop would leave.
 * Synchronises with the host (the round loop reads a convergence flag). */
int cafe_sketch_insert(void* handle, const uint32_t* gid_dev, const float* imp_dev, const int* seg_off_host, int nseg,
                       int32_t* mask_dev, int32_t* post_row_dev, int mode, void* stream);

/* Replaces SS::reset (tricks/sketch.cpp:76-116), normally triggered inside cafe_sketch_insert at a
 * call boundary; exported for tests.  Ties are ordered main table before LRU table, bucket, slot. */
int cafe_sketch_refit(void* handle, void* stream);

int cafe_sketch_sizes(void* handle, int* n1, int* n2, int* lim, int* capacity);
/* scalars[8] = threshold (float bits), real_n, num, t, flip bit, free-row FIFO length, calls so far,
 * fused-call window.  These are the members / globals of tricks/sketch.cpp:7-21. */
int cafe_sketch_scalars(void* handle, int64_t* scalars, double* decay_importance);
int cafe_sketch_set_scalars(void* handle, const int64_t* scalars, double decay_importance);
int cafe_sketch_tuning(void* handle, int window, int round_cap);
/* out[13] = calls, lookups, rounds, jobs, truncated_jobs, resets, resets_refused, flips,
 * seq_fallbacks, main_hits, lru_visits, events, max_rounds */
int cafe_sketch_stats(void* handle, int64_t* out13);
/* Full state to / from host arrays ([4*n1], [n1], [4*n2], [n2], FIFO front to back).  No counterpart
 * in tricks/sketch.cpp (its state cannot be saved); layout follows save_state/load_state of
 * TOIS_revision/PinSAGE/sketch.cpp:333-402 in spirit. */
int cafe_sketch_dump(void* handle, uint32_t* main_val, float* main_cnt, int32_t* main_dic, uint8_t* main_flip,
                     uint32_t* lru_val, float* lru_cnt, int32_t* lru_dic, int32_t* lru_t, uint8_t* lru_flip,
                     uint32_t* queue, void* stream);
int cafe_sketch_load(void* handle, const uint32_t* main_val, const float* main_cnt, const int32_t* main_dic,
                     const uint8_t* main_flip, const uint32_t* lru_val, const float* lru_cnt, const int32_t* lru_dic,
                     const int32_t* lru_t, const uint8_t* lru_flip, const uint32_t* queue, int queue_len, void* stream);

/* ---- SKEmbeddingBag data path, device ABI -------------------------------------------------------
 * Lookups are field-major: lookup p = f*B + b is sample b of field f (the reference's lS_i[F][B],
 * one id per bag).  Host arrays f_offset[nfields], hash_size[nfields], weight_hash[nfields] (device
 * pointers to [hash_size[f], D] fp32 tables); weight_high is the shared [hotn, D] hot table.
 * Row tensors are addressed as base + f*field_stride + b*sample_stride (+ column), strides in
 * floats and multiples of 4; D in {16, 32, 64, 128}. */

/* Replaces SKEmbeddingBag.query + forward (tricks/sk_embedding_bag.py:101-152): global id =
 * uint32(id + f_offset[f]); hot -> weight_high[row], else weight_hash[f][global id % hash_size[f]].
 * Also writes the global ids and the row code (-hot_row, or +hash_row) for the backward. */
int cafe_embed_forward(void* handle, const void* ids_dev, int ids_are_int64, int nfields, int B, const int64_t* f_offset,
                       const int32_t* hash_size, float* const* weight_hash, float* weight_high, int hotn, int D,
                       float* out_dev, int64_t out_field_stride, int64_t out_sample_stride, uint32_t* gid_out_dev,
                       int32_t* row_out_dev, void* stream);

/* Replaces the host-side collate of the reference's data pipeline (dlrm_data_pytorch.py:395-437: one int64 index
 * vector per field from a block of dataset rows, labels as float) for datasets in the reference's preprocessed
 * format (processed_sparse_sep.bin: int32 [N, F] sample-major, processed_label.bin: int32 [N];
 * ArtifactEvaluation/load_data.py:44-66): sparse_rows_dev is a block of B rows as it lies on disk; ids_out_dev
 * receives [F, B] field-major ids (int64 or int32), label_out_dev the labels as float (both label pointers may be
 * null).  Offsets are the implicit arange(B): one id per bag. */
int cafe_records_to_batch(const int32_t* sparse_rows_dev, int B, int F, void* ids_out_dev, int ids_are_int64,
                          const int32_t* label_dev, float* label_out_dev, void* stream);

/* cafe_embed_forward in two calls, for training.  cafe_embed_resolve is the query part alone
 * (tricks/sk_embedding_bag.py:101-113: global ids and row codes; it also keeps each lookup's bucket numbers
 * for the insert's sorts), cafe_embed_gather the two embedding_bag gathers and the where (:131-150) from the
 * row codes.  Between the two a caller can issue cafe_embed_backward_begin, whose sorts then run beside the
 * gather.  Results are identical to cafe_embed_forward. */
int cafe_embed_resolve(void* handle, const void* ids_dev, int ids_are_int64, int nfields, int B, const int64_t* f_offset,
                       const int32_t* hash_size, int hotn, uint32_t* gid_out_dev, int32_t* row_out_dev, void* stream);
int cafe_embed_gather(void* handle, const int32_t* row_dev, int nfields, int B, const int32_t* hash_size,
                      float* const* weight_hash, float* weight_high, int hotn, int D, float* out_dev,
                      int64_t out_field_stride, int64_t out_sample_stride, void* stream);

/* Replaces the importance arithmetic of insert_grad (tricks/sk_embedding_bag.py:178-189):
 * imp[p] = ||grad row p||_2 * B / sum over the field of the norms. */
int cafe_grad_importance(void* handle, const float* grad_dev, int64_t field_stride, int64_t sample_stride, int nfields,
                         int B, int D, float* imp_out_dev, void* stream);

/* No counterpart in the reference.  The same computation as cafe_grad_importance for callers that
 * cannot allocate device memory (a process whose memory pool owns the whole device, a step that must
 * not stall on an allocation): it needs no handle and allocates nothing, its intermediates live in a
 * scratch array built into the library (held by every GPU that loads it).  Limits: nfields * B <=
 * 262144 (CAFE_ERR_CAPACITY beyond that); calls on one device share the scratch, so calls that may
 * overlap on the GPU race -- issue them one after another.  The first call on a device looks up the
 * scratch address and should be made before any stream capture. */
int cafe_grad_importance_static(const float* grad_dev, int64_t field_stride, int64_t sample_stride, int nfields, int B,
                                int D, float* imp_out_dev, void* stream);

/* Replaces the row-copy loop of insert_grad (tricks/sk_embedding_bag.py:205-208), guarded: for lookups
 * with mask 1 and post_row > 0, weight_high[post_row] = weight_hash[f][local id % hash_size[f]]. */
int cafe_migrate(void* handle, const void* ids_dev, int ids_are_int64, const int32_t* mask_dev,
                 const int32_t* post_row_dev, int nfields, int B, const int64_t* f_offset, const int32_t* hash_size,
                 float* const* weight_hash, float* weight_high, int hotn, int D, int32_t* n_migrated_dev, void* stream);

/* Replaces the sparse embedding_bag backward plus torch.optim.SGD.step on weight_high and every
 * weight_hash (dlrm_s_pytorch.py:1658): row -= lr * (sum of the gradient rows of its lookups), rows
 * as coded by cafe_embed_forward. */
int cafe_scatter_sgd(void* handle, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                     const int32_t* row_dev, int nfields, int B, const int32_t* hash_size, float* const* weight_hash,
                     float* weight_high, int hotn, int D, float lr, void* stream);

/* One call for everything between loss.backward() and the end of optimizer.step() for these fields
 * (dlrm_s_pytorch.py:1653-1658): importance, insert (one reference call per field, ascending),
 * migration with pre-update rows, SGD with forward-time rows.  mask_out_dev / n_migrated_dev optional. */
int cafe_embed_backward(void* handle, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                        const void* ids_dev, int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev,
                        int nfields, int B, const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                        float* weight_high, int hotn, int D, float lr, int insert_mode, int32_t* mask_out_dev,
                        int32_t* n_migrated_dev, void* stream);

/* Optional head start for the next cafe_embed_backward / cafe_embed_backward_imp of the same lookups:
 * starts, on streams owned by the handle and ordered after `stream`, the work that needs only the
 * forward's outputs (the bucket orders of the sketch insert, the row order of the scatter), so that
 * it runs beside whatever the caller queues on `stream` in between (the dense model, an exchange of
 * gradients).  The backward recognises the head start by the same gid_dev / row_dev / sizes /
 * insert_mode and otherwise does the work itself; the two arrays must not change in between.  No
 * counterpart in the reference, whose insert is one sequential loop (sketch.cpp:268-280). */
int cafe_embed_backward_begin(void* handle, const uint32_t* gid_dev, const int32_t* row_dev, int nfields, int B,
                              const int32_t* hash_size, float* const* weight_hash, float* weight_high, int hotn, int D,
                              int insert_mode, void* stream);

/* ---- field-sharded exchange over peer memory (one node, up to 8 ranks) -----------------------------
 * No counterpart in the reference (single GPU; its --dist flags are never used, dlrm_s_pytorch.py:
 * 1090-1091).  Rank g owns the fields f with f % nranks == g (in ascending order) and serves them for
 * the global batch of nranks * rows samples.  Pointers in the *_rank / owner_* arrays are device
 * pointers valid on the calling GPU: its own buffer for its own rank, peer mappings (CUDA VMM / IPC)
 * for the others; they are accessed with ordinary loads and stores.  The caller orders the phases
 * across ranks (a stream-ordered collective between them). */

/* Every rank stores its slice ids_local[F][rows] into the owners' id buffers: owner r's buffer is
 * [F_r][nranks * rows] int64, this rank's slice at columns [rank*rows, (rank+1)*rows). */
int cafe_shard_scatter_ids(const int64_t* ids_local_dev, int nfields_total, int rows_local, int nranks, int rank,
                           int64_t* const* owner_ids, void* stream);
/* cafe_embed_forward whose output row of sample b goes to out_rank[b / rows_per_rank] at row
 * b % rows_per_rank: the all-to-all of pooled embeddings as the gather kernel's epilogue. */
int cafe_embed_forward_sharded(void* handle, const void* ids_dev, int ids_are_int64, int nfields, int B,
                               const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                               float* weight_high, int hotn, int D, float* const* out_rank, int nranks, int rows_per_rank,
                               int64_t out_field_stride, int64_t out_sample_stride, uint32_t* gid_out_dev,
                               int32_t* row_out_dev, void* stream);
/* cafe_embed_gather with the same epilogue: the row of sample b goes to out_rank[b / rows_per_rank]. */
int cafe_embed_gather_sharded(void* handle, const int32_t* row_dev, int nfields, int B, const int32_t* hash_size,
                              float* const* weight_hash, float* weight_high, int hotn, int D, float* const* out_rank,
                              int nranks, int rows_per_rank, int64_t out_field_stride, int64_t out_sample_stride,
                              void* stream);
/* The transpose for gradients, fused with cafe_grad_importance: the owner reads the gradient row of
 * sample b from grad_rank[b / rows_per_rank], writes it to local_grad_dev ([nranks*rows, nfields, D]
 * through the strides) and produces the importance array. */
int cafe_shard_pull_importance(void* handle, const float* const* grad_rank, int nranks, int rows_per_rank, int nfields,
                               int D, int64_t field_stride, int64_t sample_stride, float* local_grad_dev,
                               float* imp_out_dev, void* stream);
/* The same exchange driven from the other side (stores instead of loads over NVLink): this rank's
 * gradient buffer holds, per owner g, a block [rows, F_g, D]; each row is stored into owner g's
 * buffer owner_grad[g] ([nranks*rows, F_g, D]) at sample rank*rows + b.  The owner then runs the
 * ordinary cafe_embed_backward on its local buffer. */
int cafe_shard_push_grads(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks, int rank,
                          float* const* owner_grad, void* stream);
/* cafe_shard_push_grads for the owners' fields number j_begin .. j_end-1 only (j counts a field among its
 * owner's fields), so that the exchange can be issued in pieces and the owners can start on the first piece
 * while the next one is on its way. */
int cafe_shard_push_grads_fields(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks,
                                 int rank, float* const* owner_grad, int j_begin, int j_end, void* stream);
/* The L2 norms of the same rows, sent ahead of them (4 bytes per lookup): owner g receives them in owner_norm[g],
 * laid out [F_g, nranks*rows].  Same arithmetic as the norm step of cafe_grad_importance on the delivered rows
 * (sk_embedding_bag.py:178-184), so the owner gets the bits it would compute itself.  staging_dev: nfields_total *
 * rows_local floats of this rank's own memory. */
int cafe_shard_push_norms(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks, int rank,
                          float* const* owner_norm, float* staging_dev, void* stream);
/* cafe_embed_backward from norms that are already there (cafe_shard_push_norms) while the gradient rows may still be
 * on their way: importance (sk_embedding_bag.py:185-189), sketch insert and migration run at once; the stream waits
 * for gate_event (a cudaEvent_t, or null) only before the SGD scatter, the one step that reads the rows.  Results
 * are those of cafe_embed_backward on the delivered rows. */
int cafe_embed_backward_norms(void* handle, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                              const float* norm_dev, const void* ids_dev, int ids_are_int64, const uint32_t* gid_dev,
                              const int32_t* row_dev, int nfields, int B, const int64_t* f_offset, const int32_t* hash_size,
                              float* const* weight_hash, float* weight_high, int hotn, int D, float lr, int insert_mode,
                              void* gate_event, void* stream);
/* cafe_embed_backward whose gradient rows of the fields from gate_field on are still being written when the call
 * is made: they are complete once gate_event (a cudaEvent_t) has fired.  The fields before gate_field are
 * processed at once; the importance of the late fields is computed behind the gate on a stream of the handle,
 * and the insert, which takes the fields in ascending order like the reference's per-field calls
 * (sk_embedding_bag.py:173-208 called per table), waits for it only when it gets there.  Results are those of
 * cafe_embed_backward.  No counterpart in the reference (single GPU). */
int cafe_embed_backward_gated(void* handle, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                              const void* ids_dev, int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev,
                              int nfields, int B, const int64_t* f_offset, const int32_t* hash_size,
                              float* const* weight_hash, float* weight_high, int hotn, int D, float lr, int insert_mode,
                              int gate_field, void* gate_event, void* stream);
/* cafe_embed_backward for a caller that already holds the importance array. */
int cafe_embed_backward_imp(void* handle, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                            const float* imp_dev, const void* ids_dev, int ids_are_int64, const uint32_t* gid_dev,
                            const int32_t* row_dev, int nfields, int B, const int64_t* f_offset, const int32_t* hash_size,
                            float* const* weight_hash, float* weight_high, int hotn, int D, float lr, int insert_mode,
                            int32_t* mask_out_dev, void* stream);

/* ---- the one-stage HotSketch of the artifact tree, device ABI -----------------------------------------
 * Replaces class SS of ArtifactEvaluation/embeddings/sketch.cpp (the sketch of the SIGMOD'24 paper; the
 * reference keeps one per field in ss[26], :151, selected by the `idx` argument of its entry points --
 * here every sketch is a handle).  Device pointers, caller-owned outputs, no synchronisation except in
 * dump / load. */
/* init(n, Threshold, dr, idx), sketch.cpp:228-230: lim buckets, rows 1..lim-1 free. */
int cafe_sigmod_create(void** handle_out, int lim, int threshold, double decay_rate, int max_lookups);
int cafe_sigmod_destroy(void* handle);
/* batch_query, sketch.cpp:124-130: out[i] = -row if the id holds a hot row, else (int32)id. */
int cafe_sigmod_query(void* handle, const uint32_t* gid_dev, int n, int32_t* out_dev, void* stream);
/* batch_insert_val / batch_insert (imp_dev null), sketch.cpp:131-149: decay check, then Insert per lookup in
 * order; mask_out_dev[i] = 1 where the lookup was handed a hot row. */
int cafe_sigmod_insert(void* handle, const uint32_t* gid_dev, const float* imp_dev, int n, int32_t* mask_out_dev,
                       void* stream);
/* update(idx), sketch.cpp:61-75, 222-225: rebuild the free-row FIFO from the rows the buckets hold. */
int cafe_sigmod_update(void* handle, void* stream);
/* The query of SKEmbeddingBag.forward (ArtifactEvaluation/embeddings/sk_embedding_bag.py:77-88, 95-118) for one
 * field: global ids and row codes (-hot row, or global id % hash_size) for cafe_embed_gather / cafe_scatter_sgd. */
int cafe_sigmod_resolve(void* handle, const void* ids_dev, int ids_are_int64, int64_t f_offset, int hash_size, int n,
                        uint32_t* gid_out_dev, int32_t* row_out_dev, void* stream);
/* The post-insert query of insert_grad (sk_embedding_bag.py:173-180): hot row of every lookup with mask 1
 * (0 elsewhere), the post_row input of cafe_migrate. */
int cafe_sigmod_post_rows(void* handle, const uint32_t* gid_dev, const int32_t* mask_dev, int n, int32_t* post_row_out_dev,
                          void* stream);
/* State export / import with host arrays (val, cnt, dic: 4 * lim each; queue: lim; scalars[0..2] = rows handed
 * out, FIFO length, decays).  The reference saves nothing and calls update() after loading the model
 * (ArtifactEvaluation/main.py); load restores the buckets and rebuilds the FIFO the same way. */
int cafe_sigmod_dump(void* handle, uint32_t* val, float* cnt, int32_t* dic, uint32_t* queue, int64_t* scalars, double* tot,
                     void* stream);
int cafe_sigmod_load(void* handle, const uint32_t* val, const float* cnt, const int32_t* dic, int64_t num, double tot,
                     void* stream);
/* Workspace of the embedding entry points (cafe_grad_importance, cafe_embed_gather, cafe_migrate, cafe_scatter_sgd)
 * for a model whose sketch is not the CAFE+ one: a handle without a sketch.  No counterpart in the reference
 * (its modules allocate through torch).  Destroy with cafe_sketch_destroy. */
int cafe_workspace_create(void** handle_out, int hotn, int max_lookups);

/* ---- the reference's own ctypes ABI, host pointers (tricks/sketch.cpp:300-327) ------------------
 * Same names, argument meaning and result convention (pointer to a library-owned int array that is
 * valid until the next call), so that the reference's Python can bind this library in place of its
 * sklib.so.  One process-global sketch; data are staged through device buffers.  On failure the
 * pointer-returning calls return NULL and the double-returning calls return -1 (see
 * cafe_last_error). */
void init(int n, int Threshold, int adjust_thres, double alp);
int* batch_query(uint32_t* data, int len);
int* batch_insert(uint32_t* data, int len);
int* batch_insert_val(uint32_t* data, float* v, int len);
double analyse(uint32_t* data, int len);
double analyse1(uint32_t* data, int len);
/* The handle behind the six calls above (NULL before init), for use with the device ABI. */
void* cafe_global_handle(void);
/* Largest len the six calls accept (default 1<<21); takes effect at the next init. */
int cafe_global_set_capacity(int max_len);

/* ---- measurement ---------------------------------------------------------------------------------
 * No counterpart in the reference.  Kernel launches of the library are always counted per slot;
 * with cafe_profile_enable(1) each launch is also bracketed by CUDA events on its stream.
 * cafe_profile_read fills ms[slots] (event time summed per slot) and launches[slots] since the last
 * read, after synchronising the device. */
int cafe_profile_slots(void);
const char* cafe_profile_slot_name(int slot);
int cafe_profile_enable(int on);
int cafe_profile_read(double* ms_out, int64_t* launches_out);
int64_t cafe_launch_count(void);

/* ---- DLRM's dot interaction (dlrm_s_pytorch.py:779-812, `interact_features` with arch_interaction_op "dot") --------
 * One kernel per direction instead of cat + bmm + two index gathers + cat.  x_dev [B, D] is the bottom MLP's output (null:
 * no dense vector, as in the Avazu models); vector f of sample b of the pooled embeddings lies at emb_dev + b *
 * sample_stride + f * field_stride (so the [B, F, D] output of cafe_embed_forward is read in place); out_dev [B,
 * out_stride] receives { x | T_i . T_j for i ascending, j < i (itself = 0) or j <= i (itself = 1) }, T = { x, the F
 * vectors }: the reference's order (:800-812).  F + 1 <= 64, D <= 128, fp32.  Status 6 if the sample does not fit
 * 48 KB of shared memory. */
int cafe_dot_interaction_forward(const float* x_dev, const float* emb_dev, int64_t field_stride, int64_t sample_stride, int B,
                                 int F, int D, int itself, float* out_dev, int64_t out_stride, void* stream);
/* Its backward: grad_x_dev [B, D] (when x_dev was given; includes the pass-through of the leading D columns) and the
 * gradient of every embedding vector at grad_emb_dev + b * gsample_stride + f * gfield_stride. */
int cafe_dot_interaction_backward(const float* x_dev, const float* emb_dev, int64_t field_stride, int64_t sample_stride, int B,
                                  int F, int D, int itself, const float* grad_out_dev, int64_t out_stride, float* grad_x_dev,
                                  float* grad_emb_dev, int64_t gfield_stride, int64_t gsample_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CAFE_B200_H */
