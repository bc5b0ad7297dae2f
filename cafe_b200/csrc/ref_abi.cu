// ref_abi.cu -- the reference's ctypes ABI (tricks/sketch.cpp:300-327) on top of the device sketch.
//
// The six symbols keep the reference's names and calling convention (host pointers in, pointer to a
// library-owned int array out), so the reference's Python binds this library unchanged.  Inputs are
// staged to the device, the device sketch does the work, results are staged back.
#include <cuda_runtime.h>
#include <stdio.h>

#include <vector>

#include "../../include/cafe_b200.h"
#include "cafe_internal.h"
#include "sketch_core.cuh"

static void* g_handle = nullptr;
static int g_cap = 1 << 21;
static int g_alloc = 0;
static uint32_t* g_ids = nullptr;
static float* g_val = nullptr;
static int32_t* g_out = nullptr;
static int32_t* g_count = nullptr;
static std::vector<int32_t> g_ins, g_que;

__global__ void k_count(const CafeMainBucket* __restrict__ mb, int n1, const uint32_t* __restrict__ gid, int n,
                        int any_slot, int32_t* __restrict__ count) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t x = gid[i];
    const CafeMainBucket& b = mb[cafe_hash(x, n1)];
    int hit = 0;
    if (any_slot) {   // SS::Query, sketch.cpp:142-150
        for (int s = 0; s < CAFE_SLOTS; ++s) hit |= (b.val[s] == x);
    } else {          // query() < 0, sketch.cpp:314-319
        hit = cafe_probe_hot(b, x) != 0;
    }
    if (hit) atomicAdd(count, 1);
}

static bool stage(const uint32_t* data, const float* v, int len) {
    if (!g_handle) { cafe_internal_set_error("init() has not been called"); return false; }
    if (len < 0 || len > g_alloc || (len > 0 && !data)) { cafe_internal_set_error("len exceeds the staging capacity"); return false; }
    if (len == 0) return true;
    if (cudaMemcpy(g_ids, data, 4 * (size_t)len, cudaMemcpyHostToDevice) != cudaSuccess) return false;
    if (v && cudaMemcpy(g_val, v, 4 * (size_t)len, cudaMemcpyHostToDevice) != cudaSuccess) return false;
    return true;
}

static int* insert_common(uint32_t* data, float* v, int len) {
    if (!stage(data, v, len)) return nullptr;
    int seg[2] = {0, len};
    int rc = cafe_sketch_insert(g_handle, g_ids, v ? g_val : nullptr, seg, 1, g_out, nullptr, CAFE_INSERT_PARALLEL, 0);
    if (rc != CAFE_OK && rc != CAFE_ERR_NOCONVERGE && rc != CAFE_ERR_RESET_UNDERFLOW) return nullptr;
    if (len > 0 && cudaMemcpy(g_ins.data(), g_out, 4 * (size_t)len, cudaMemcpyDeviceToHost) != cudaSuccess) return nullptr;
    return g_ins.data();
}

static double count_common(uint32_t* data, int len, int any_slot) {
    if (len <= 0 || !stage(data, nullptr, len)) return -1.0;
    CafeSketchView V = cafe_internal_view(g_handle);
    cudaMemset(g_count, 0, 4);
    k_count<<<(len + 255) / 256, 256>>>(V.main, V.n1, g_ids, len, any_slot, g_count);
    int32_t c = 0;
    if (cudaMemcpy(&c, g_count, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1.0;
    return 1.0 * c / len;
}

extern "C" {

void* cafe_global_handle(void) { return g_handle; }

int cafe_global_set_capacity(int max_len) {
    if (max_len < 1) return CAFE_ERR_ARG;
    g_cap = max_len;
    return CAFE_OK;
}

void init(int n, int Threshold, int adjust_thres, double alp) {
    if (g_handle) { cafe_sketch_destroy(g_handle); g_handle = nullptr; }
    if (g_ids) { cudaFree(g_ids); cudaFree(g_val); cudaFree(g_out); cudaFree(g_count); g_ids = nullptr; }
    g_alloc = 0;
    if (cafe_sketch_create(&g_handle, n, (float)Threshold, adjust_thres, alp, g_cap) != CAFE_OK) {
        fprintf(stderr, "cafe_b200 init failed: %s\n", cafe_last_error());
        g_handle = nullptr;
        return;
    }
    if (cudaMalloc(&g_ids, 4 * (size_t)g_cap) != cudaSuccess || cudaMalloc(&g_val, 4 * (size_t)g_cap) != cudaSuccess ||
        cudaMalloc(&g_out, 4 * (size_t)g_cap) != cudaSuccess || cudaMalloc(&g_count, 4) != cudaSuccess) {
        fprintf(stderr, "cafe_b200 init failed: staging buffers\n");
        cafe_sketch_destroy(g_handle);
        g_handle = nullptr;
        return;
    }
    g_alloc = g_cap;
    g_ins.assign((size_t)g_cap, 0);
    g_que.assign((size_t)g_cap, 0);
}

int* batch_query(uint32_t* data, int len) {
    if (!stage(data, nullptr, len)) return nullptr;
    if (cafe_sketch_query(g_handle, g_ids, len, g_out, 0) != CAFE_OK) return nullptr;
    if (len > 0 && cudaMemcpy(g_que.data(), g_out, 4 * (size_t)len, cudaMemcpyDeviceToHost) != cudaSuccess) return nullptr;
    return g_que.data();
}

int* batch_insert(uint32_t* data, int len) { return insert_common(data, nullptr, len); }

int* batch_insert_val(uint32_t* data, float* v, int len) {
    if (len > 0 && !v) { cafe_internal_set_error("null importance array"); return nullptr; }
    return insert_common(data, v, len);
}

double analyse(uint32_t* data, int len) { return count_common(data, len, 0); }
double analyse1(uint32_t* data, int len) { return count_common(data, len, 1); }

}  // extern "C"
