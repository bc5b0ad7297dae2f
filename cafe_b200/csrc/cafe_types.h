// cafe_types.h -- data layout of the device-resident HotSketch and shared constants.
//
// The reference keeps one 52-byte main bucket and one 68-byte LRU bucket per hash value
// (tricks/sketch.cpp:23-35).  Here both are padded to 16-byte multiples and ordered so that the two
// fields a query needs (val, dic) share the first 32-byte sector of a 64-byte main bucket.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define CAFE_HD __host__ __device__ __forceinline__
#else
#define CAFE_HD inline
#endif

#define CAFE_SLOTS 4
#define CAFE_MAX_SEGMENTS 64   // fields handled by one fused insert

// status codes returned by every C entry point (0 = ok); same values as include/cafe_b200.h
#ifndef CAFE_STATUS_ENUMS
#define CAFE_STATUS_ENUMS
enum {
    CAFE_OK = 0,
    CAFE_ERR_ARG = 1,          // null pointer, negative size, bad handle
    CAFE_ERR_CAPACITY = 2,     // request larger than the handle or a static buffer was sized for
    CAFE_ERR_CUDA = 3,         // a CUDA runtime call failed (see cafe_last_error)
    CAFE_ERR_NOCONVERGE = 4,   // parallel insert hit its round cap (the sequential kernel was used)
    CAFE_ERR_RESET_UNDERFLOW = 5, // threshold re-fit refused: fewer candidates than hot rows
    CAFE_ERR_UNSUPPORTED = 6
};
enum { CAFE_INSERT_PARALLEL = 0, CAFE_INSERT_SEQUENTIAL = 1 };
#endif

struct alignas(16) CafeMainBucket {   // 64 B
    uint32_t val[CAFE_SLOTS];
    int32_t dic[CAFE_SLOTS];
    float cnt[CAFE_SLOTS];
    uint32_t flip;
    uint32_t pad[3];
};

struct alignas(16) CafeLruBucket {    // 80 B
    uint32_t val[CAFE_SLOTS];
    int32_t dic[CAFE_SLOTS];
    float cnt[CAFE_SLOTS];
    int32_t t[CAFE_SLOTS];
    uint32_t flip;
    uint32_t pad[3];
};

// A promotion into the main table caused by the lookup at one batch position.
enum { CAFE_EV_NONE = 0, CAFE_EV_OWN = 2, CAFE_EV_VICTIM = 3 };
struct alignas(16) CafeEvent {
    uint32_t x;      // id that moves to the main table
    float cnt;       // its count
    int32_t dic;     // the hot row it carries (0 = none)
    uint32_t kind;   // CAFE_EV_*
};

// Totals one round of the parallel insert reports to the host.
struct CafeRoundResult {
    int32_t changed;       // beliefs consumed this round differ from the ones it produced
    int32_t tl_changed;    // ... in particular the FIFO timeline
    int32_t n_miss;        // lookups that went to the LRU stage
    int32_t num_delta;     // hot rows handed out
    int32_t n_pop_ok;      // successful pops of the free-row FIFO
    int32_t n_push;        // pushes to the free-row FIFO
    int32_t error;         // internal consistency problems seen (0 = none)
    int32_t n_main_hit;
    int32_t n_events;
    int32_t miss_changed;  // the main pass of this round sent a lookup to the LRU stage that was not there before, or took one away
    int32_t list_cursor[3];  // work counters of the launches that go through the long-bucket lists (main, LRU, final pass)
    int32_t seg_real_delta[CAFE_MAX_SEGMENTS];  // change of real_n per segment
};
