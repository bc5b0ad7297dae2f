// prof.cu -- per-kernel timing with CUDA events on the launching stream, and launch counting.
//
// Every kernel launch (or CUB call) of the library is bracketed by cafe_prof_begin / cafe_prof_end
// with a slot id.  Launches are always counted; when profiling is switched on, an event pair is
// recorded around each one and cafe_profile_read() sums the elapsed times per slot.
#include <cuda_runtime.h>

#include <vector>

#include "../../include/cafe_b200.h"
#include "cafe_internal.h"

static const char* kSlotNames[CAFE_PROF_SLOTS] = {
    "embed_forward", "grad_norm", "field_sum", "importance", "lookup_hash_sort", "main_pass", "miss_scan", "lru_pass",
    "fifo_resolve", "fifo_commit", "threshold_refit", "migrate", "row_keys", "row_sort", "scatter_chunks",
    "scatter_fixup", "seq_insert", "query", "memset", "other", "main_pass_later_rounds", "main_pass_final",
    "lru_pass_later_rounds", "push_grads", "scatter_ids"};

struct Rec { int slot; cudaEvent_t e0, e1; };
static bool g_on = false;
static std::vector<cudaEvent_t> g_pool;
static std::vector<Rec> g_recs;
static int64_t g_launches[CAFE_PROF_SLOTS];
static int64_t g_total_launches = 0;
static Rec* g_open = nullptr;

// While per-kernel timing is on, the library queues its side-stream work on the caller's stream so
// that every event pair brackets one kernel running alone.
bool cafe_prof_serialise() { return g_on; }

static cudaEvent_t take_event() {
    if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
    cudaEvent_t e;
    cudaEventCreate(&e);
    return e;
}

void cafe_prof_begin(int slot, cudaStream_t st) {
    ++g_launches[slot];
    ++g_total_launches;
    if (!g_on) return;
    Rec r;
    r.slot = slot;
    r.e0 = take_event();
    r.e1 = take_event();
    cudaEventRecord(r.e0, st);
    g_recs.push_back(r);
    g_open = &g_recs.back();
}
void cafe_prof_end(cudaStream_t st) {
    if (!g_on || !g_open) return;
    cudaEventRecord(g_open->e1, st);
    g_open = nullptr;
}

extern "C" {

int cafe_profile_slots(void) { return CAFE_PROF_SLOTS; }
const char* cafe_profile_slot_name(int i) { return (i >= 0 && i < CAFE_PROF_SLOTS) ? kSlotNames[i] : ""; }

int cafe_profile_enable(int on) {
    g_on = on != 0;
    return CAFE_OK;
}

// ms_out[slots] += summed event time per slot since the last read; launches_out[slots] = launches
// since the last read (counted whether or not timing was on).  Synchronises the device.
int cafe_profile_read(double* ms_out, int64_t* launches_out) {
    if (cudaDeviceSynchronize() != cudaSuccess) return CAFE_ERR_CUDA;
    for (int i = 0; i < CAFE_PROF_SLOTS; ++i) {
        if (ms_out) ms_out[i] = 0.0;
        if (launches_out) launches_out[i] = g_launches[i];
        g_launches[i] = 0;
    }
    for (Rec& r : g_recs) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess && ms_out) ms_out[r.slot] += ms;
        g_pool.push_back(r.e0);
        g_pool.push_back(r.e1);
    }
    g_recs.clear();
    g_open = nullptr;
    return CAFE_OK;
}

int64_t cafe_launch_count(void) { return g_total_launches; }

}  // extern "C"
