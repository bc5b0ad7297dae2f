// cafe_internal.h -- declarations shared by the translation units of libcafe_b200 (not installed).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "cafe_types.h"


#define CAFE_MAX_DIM 128      // widest embedding row the scatter workspace is sized for
#define CAFE_CHUNK 32         // sorted lookups reduced by one thread group in the scatter

struct CafeSketchView {
    const CafeMainBucket* main;
    int n1, lim, cap;
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
    int32_t* pos[2] = {nullptr, nullptr};    // [cap] lookup position, unsorted / sorted
    float* partial = nullptr;    // [2 * ceil(cap/CAFE_CHUNK) * CAFE_MAX_DIM] partial row sums of chunk-spanning rows
    void* cub_tmp = nullptr;
    size_t cub_bytes = 0;
};

int cafe_embed_ws_init(CafeEmbedWorkspace* ws, int cap, int hotn);
void cafe_embed_ws_free(CafeEmbedWorkspace* ws);

CafeSketchView cafe_internal_view(void* h);
CafeEmbedWorkspace* cafe_internal_ws(void* h);
int cafe_internal_insert(void* h, const uint32_t* gid, const float* imp, const int* seg_off, int nseg, int32_t* mask,
                         int32_t* post_row, int mode, cudaStream_t stream);
void cafe_internal_set_error(const char* msg);
