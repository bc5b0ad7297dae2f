// cafe_internal.h -- declarations shared by the translation units of libcafe_b200 (not installed).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "cafe_types.h"


#define CAFE_MAX_DIM 128      // widest embedding row the scatter workspace is sized for
#define CAFE_CHUNK 32         // sorted lookups reduced by one thread group in the scatter

struct CafeSketchView {
    const CafeMainBucket* main;
    int n1, n2, lim, cap;
};

// Device buffers of the embedding path, sized once per handle for `cap` lookups.
struct CafeEmbedWorkspace {
    int cap = 0;
    float* norm = nullptr;       // [cap] gradient norm per lookup
    float* imp = nullptr;        // [cap] importance per lookup
    float* totals = nullptr;     // [CAFE_MAX_SEGMENTS] sum of norms per field
    int32_t* mask = nullptr;     // [cap] newly-hot flag per lookup
    int32_t* post_row = nullptr; // [cap] hot row after the lookup's own call
    uint32_t* key[2] = {nullptr, nullptr};   // [cap] unified row key, unsorted / sorted
    int32_t* pos[2] = {nullptr, nullptr};    // [cap] lookup position: intermediate pass of the sort / sorted
    float* partial = nullptr;    // [2 * ceil(cap/CAFE_CHUNK) * CAFE_MAX_DIM] partial row sums of chunk-spanning rows
    int32_t* row_winner = nullptr;   // [hotn] migration: highest position that claims a hot row in this call (-1 between calls)
    uint32_t* key_tmp = nullptr;     // [cap] intermediate keys of the row sort
    uint32_t* bucket_key[2] = {nullptr, nullptr};   // [cap] main / LRU bucket of every lookup, left by cafe_embed_resolve ...
    const uint32_t* keys_of = nullptr;              // ... for the lookups whose global ids are in this array
    int keys_total = 0;
    int32_t* sort_scratch = nullptr; // radix-sort histograms
    cudaStream_t side = nullptr;     // runs the scatter's key sort beside the sketch insert
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaStream_t late = nullptr;     // importance of fields whose gradients arrive behind a gate
    cudaEvent_t ev_late = nullptr;
    // arrays whose side work cafe_embed_backward_begin has already started (null: none)
    const uint32_t* begun_gid = nullptr;
    const int32_t* begun_row = nullptr;
    int begun_total = 0, begun_mode = 0;
};

int cafe_embed_ws_init(CafeEmbedWorkspace* ws, int cap, int hotn);
void cafe_embed_ws_free(CafeEmbedWorkspace* ws);

CafeSketchView cafe_internal_view(void* h);
CafeEmbedWorkspace* cafe_internal_ws(void* h);
int cafe_internal_insert(void* h, const uint32_t* gid, const float* imp, const int* seg_off, int nseg, int32_t* mask,
                         int32_t* post_row, int mode, cudaStream_t stream);
// starts the insert's bucket sorts of `gid` beside whatever the caller queues next on `stream`
// (key1 / key2: the lookups' main / LRU bucket numbers if the caller has them, else null)
void cafe_internal_presort(void* h, const uint32_t* gid, int n, const uint32_t* key1, const uint32_t* key2, cudaStream_t stream);
// counts of segments >= seg of the next cafe_internal_insert are valid once `ev` has fired (null: no gate)
void cafe_internal_set_gate(void* h, int seg, cudaEvent_t ev);
void cafe_internal_set_error(const char* msg);

// ---- per-kernel timing and launch counting (prof.cu) ------------------------------------------------
enum {
    CAFE_P_FORWARD = 0, CAFE_P_NORM, CAFE_P_FIELDSUM, CAFE_P_IMPORTANCE, CAFE_P_LOOKUP_SORT, CAFE_P_MAIN, CAFE_P_SCAN,
    CAFE_P_LRU, CAFE_P_RESOLVE, CAFE_P_COMMIT, CAFE_P_REFIT, CAFE_P_MIGRATE, CAFE_P_ROWKEYS, CAFE_P_ROWSORT,
    CAFE_P_SCATTER, CAFE_P_FIXUP, CAFE_P_SEQ, CAFE_P_QUERY, CAFE_P_MEMSET, CAFE_P_OTHER, CAFE_P_MAIN_LATER, CAFE_P_MAIN_FINAL,
    CAFE_P_LRU_LATER, CAFE_P_PUSH, CAFE_P_IDS, CAFE_PROF_SLOTS
};
bool cafe_prof_serialise();
void cafe_prof_begin(int slot, cudaStream_t st);
void cafe_prof_end(cudaStream_t st);
struct CafeProfScope {
    cudaStream_t st;
    CafeProfScope(int slot, cudaStream_t s) : st(s) { cafe_prof_begin(slot, s); }
    ~CafeProfScope() { cafe_prof_end(st); }
};
#define CAFE_PROF(slot, stream) CafeProfScope cafe_prof_scope_##slot(slot, stream)
#define CAFE_PROF_DYN(slot, stream) CafeProfScope cafe_prof_scope_dyn(slot, stream)
