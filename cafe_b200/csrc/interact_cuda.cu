// interact_cuda.cu -- the dot interaction of DLRM (dlrm_s_pytorch.py:779-812, `interact_features`, "dot") as one
// kernel per direction.  The reference concatenates the dense vector and the F pooled embedding vectors of a sample
// into T [(F+1), D], forms Z = T T^t with a batched matrix product, picks the entries below the diagonal (or on and
// below it with arch_interaction_itself) through two index lists and concatenates them behind the dense vector:
// four launches, a [B, F+1, F+1] intermediate and a gather per direction.  Here a block takes one sample: the F+1
// vectors are staged in shared memory once, every thread computes a few of the dot products and writes them to their
// place in the output row; the backward forms the symmetric weight matrix of the sample from the incoming gradient
// and multiplies it back onto the staged vectors.  27 x 27 x 128 multiply-adds per sample: no tensor cores needed.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cafe_b200.h"
#include "cafe_internal.h"

#define CAFE_INTERACT_MAX_VECS 64   // F + 1
#define CAFE_INTERACT_THREADS 128

// pair number p of (i, j), j < i + off (off = 1: the diagonal counts), in the reference's order: i ascending, j ascending
__device__ __forceinline__ int cafe_pair_index(int i, int j, int off) { return i * (i - 1 + 2 * off) / 2 + j; }

// x [B, D] (dense vector; may be null: no dense vector, F vectors only), emb: vector f of sample b at
// emb + b * sample_stride + f * field_stride, out [B, out_stride] = { x (if given) | pairs }
__global__ void __launch_bounds__(CAFE_INTERACT_THREADS)
k_interact_forward(const float* __restrict__ x, const float* __restrict__ emb, int64_t field_stride, int64_t sample_stride, int F,
                   int D, int off, float* __restrict__ out, int64_t out_stride) {
    extern __shared__ float sh[];
    const int nv = F + (x ? 1 : 0);
    const int ld = D + 1;   // row pitch: two rows never start in the same bank
    float* T = sh;
    const int64_t b = blockIdx.x;
    for (int e = threadIdx.x; e < nv * D; e += blockDim.x) {
        const int v = e / D, d = e - v * D;
        float val;
        if (x && v == 0) val = x[b * D + d];
        else val = emb[b * sample_stride + (int64_t)(v - (x ? 1 : 0)) * field_stride + d];
        T[v * ld + d] = val;
    }
    __syncthreads();
    float* o = out + b * out_stride;
    const int lead = x ? D : 0;
    for (int d = threadIdx.x; d < lead; d += blockDim.x) o[d] = T[d];
    const int npairs = cafe_pair_index(nv, 0, off);
    for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
        // (i, j) of pair p: the largest i whose first pair number is <= p
        int i = off ? 0 : 1;
        while (cafe_pair_index(i + 1, 0, off) <= p) ++i;
        const int j = p - cafe_pair_index(i, 0, off);
        const float* a = T + i * ld;
        const float* c = T + j * ld;
        float s = 0.f;
        for (int d = 0; d < D; ++d) s += a[d] * c[d];
        o[lead + p] = s;
    }
}

// grad_out [B, out_stride] -> grad_x [B, D] (if x was given), grad_emb (same addressing as emb)
__global__ void __launch_bounds__(CAFE_INTERACT_THREADS)
k_interact_backward(const float* __restrict__ x, const float* __restrict__ emb, int64_t field_stride, int64_t sample_stride, int F,
                    int D, int off, const float* __restrict__ grad_out, int64_t out_stride, float* __restrict__ grad_x,
                    float* __restrict__ grad_emb, int64_t gfield_stride, int64_t gsample_stride) {
    extern __shared__ float sh[];
    const int nv = F + (x ? 1 : 0);
    const int ld = D + 1;
    float* T = sh;                       // [nv][ld]
    float* G = sh + nv * ld;             // [nv][nv]: d(loss)/d(T_i . T_j), symmetric; the diagonal doubled
    const int64_t b = blockIdx.x;
    for (int e = threadIdx.x; e < nv * D; e += blockDim.x) {
        const int v = e / D, d = e - v * D;
        float val;
        if (x && v == 0) val = x[b * D + d];
        else val = emb[b * sample_stride + (int64_t)(v - (x ? 1 : 0)) * field_stride + d];
        T[v * ld + d] = val;
    }
    const float* g = grad_out + b * out_stride;
    const int lead = x ? D : 0;
    for (int e = threadIdx.x; e < nv * nv; e += blockDim.x) {
        const int i = e / nv, j = e - i * nv;
        float w = 0.f;
        if (j < i) w = g[lead + cafe_pair_index(i, j, off)];
        else if (j > i) w = g[lead + cafe_pair_index(j, i, off)];
        else if (off) w = 2.0f * g[lead + cafe_pair_index(i, i, off)];
        G[e] = w;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nv * D; e += blockDim.x) {
        const int i = e / D, d = e - i * D;
        float s = 0.f;
        for (int j = 0; j < nv; ++j) s += G[i * nv + j] * T[j * ld + d];
        if (x && i == 0) grad_x[b * D + d] = s + g[d];
        else grad_emb[b * gsample_stride + (int64_t)(i - (x ? 1 : 0)) * gfield_stride + d] = s;
    }
}

extern "C" {

static int interact_args_ok(const float* emb, int B, int F, int D, int itself, int64_t fs, int64_t ss) {
    if (B < 0 || F < 1 || F + 1 > CAFE_INTERACT_MAX_VECS || D < 1 || D > CAFE_MAX_DIM || (itself != 0 && itself != 1)) return 0;
    if (B > 0 && (!emb || fs < D || ss < D)) return 0;
    return 1;
}

int cafe_dot_interaction_forward(const float* x_dev, const float* emb_dev, int64_t field_stride, int64_t sample_stride, int B,
                                 int F, int D, int itself, float* out_dev, int64_t out_stride, void* stream) {
    if (!interact_args_ok(emb_dev, B, F, D, itself, field_stride, sample_stride)) return CAFE_ERR_ARG;
    const int nv = F + (x_dev ? 1 : 0);
    const int npairs = nv * (nv - 1 + 2 * itself) / 2;
    if (B == 0) return CAFE_OK;
    if (!out_dev || out_stride < (x_dev ? D : 0) + npairs) return CAFE_ERR_ARG;
    const size_t smem = sizeof(float) * (size_t)nv * (D + 1);
    if (smem > 48 * 1024) return CAFE_ERR_UNSUPPORTED;
    k_interact_forward<<<B, CAFE_INTERACT_THREADS, smem, (cudaStream_t)stream>>>(x_dev, emb_dev, field_stride, sample_stride, F, D,
                                                                                itself, out_dev, out_stride);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { cafe_internal_set_error(cudaGetErrorString(e)); return CAFE_ERR_CUDA; }
    return CAFE_OK;
}

int cafe_dot_interaction_backward(const float* x_dev, const float* emb_dev, int64_t field_stride, int64_t sample_stride, int B,
                                  int F, int D, int itself, const float* grad_out_dev, int64_t out_stride, float* grad_x_dev,
                                  float* grad_emb_dev, int64_t gfield_stride, int64_t gsample_stride, void* stream) {
    if (!interact_args_ok(emb_dev, B, F, D, itself, field_stride, sample_stride)) return CAFE_ERR_ARG;
    if (B == 0) return CAFE_OK;
    if (!grad_out_dev || !grad_emb_dev || (x_dev && !grad_x_dev) || gfield_stride < D || gsample_stride < D) return CAFE_ERR_ARG;
    const int nv = F + (x_dev ? 1 : 0);
    const size_t smem = sizeof(float) * ((size_t)nv * (D + 1) + (size_t)nv * nv);
    if (smem > 48 * 1024) return CAFE_ERR_UNSUPPORTED;
    k_interact_backward<<<B, CAFE_INTERACT_THREADS, smem, (cudaStream_t)stream>>>(x_dev, emb_dev, field_stride, sample_stride, F, D,
                                                                                 itself, grad_out_dev, out_stride, grad_x_dev,
                                                                                 grad_emb_dev, gfield_stride, gsample_stride);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { cafe_internal_set_error(cudaGetErrorString(e)); return CAFE_ERR_CUDA; }
    return CAFE_OK;
}

}  // extern "C"
