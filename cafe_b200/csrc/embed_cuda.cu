// embed_cuda.cu -- the SKEmbeddingBag data path on sm_100a: fused query+gather forward, gradient-norm
// importance, hot-row migration, and sort/segment-reduce scatter with the SGD update in place.
//
// Reference being replaced (tricks/sk_embedding_bag.py): query + two embedding_bag gathers + where
// (:101-152), importance from gradient norms (:173-190), migration of newly-hot ids (:199-208), and the
// sparse SGD step of the caller (dlrm_s_pytorch.py:1658).  All of it is HBM-bound gather/scatter work:
// rows move as 16-byte vectors, one group of D/4 lanes per row, no tensor cores.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "../../include/cafe_b200.h"
#include "cafe_internal.h"
#include "radix_sort.cuh"
#include "sketch_core.cuh"

struct CafeFields {
    int32_t nfields, B, D, hotn;
    uint32_t f_offset[CAFE_MAX_SEGMENTS];   // added to a field's local id to give the global id
    int32_t hash_size[CAFE_MAX_SEGMENTS];
    int32_t hash_base[CAFE_MAX_SEGMENTS + 1];   // prefix sums of hash_size (unified row numbering)
    float* w_hash[CAFE_MAX_SEGMENTS];
    float* w_high;
};

// Where the rows of a batch go (forward) or come from (backward) when the batch is spread over the
// GPUs of a node: sample b belongs to rank b / rows_per_rank, whose buffer starts at base[rank]
// (this GPU's own memory for its own slice, a peer mapping for the others).  One rank: base[0], all rows.
#define CAFE_MAX_RANKS 8
struct CafeRankBuffers {
    float* base[CAFE_MAX_RANKS];
    int32_t rows_per_rank;
};

#define FULL 0xffffffffu

__device__ __forceinline__ float4 ld_row(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ld_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

template <typename T>
__device__ __forceinline__ T* shfl_ptr(T* p, int src) {
    return reinterpret_cast<T*>(__shfl_sync(FULL, reinterpret_cast<unsigned long long>(p), src));
}

// ---------------------------------------------------------------------------------------------
// forward: per lookup, probe the sketch (hot row or hash row), then copy the selected row.
// A warp first resolves 32 lookups (32 independent bucket reads in flight), then its lanes move
// the 32 rows, G = D/4 lanes per row, 4 rows' loads issued before their stores.
// ---------------------------------------------------------------------------------------------
template <int G, typename IdT>
__global__ void __launch_bounds__(256)
k_embed_forward(const __grid_constant__ CafeFields F, const IdT* __restrict__ ids,
                const CafeMainBucket* __restrict__ mb, int n1, const CafeRankBuffers out, int64_t field_stride,
                int64_t sample_stride, uint32_t* __restrict__ gid_out, int32_t* __restrict__ row_out, int total) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t p = warp * 32 + lane;
    const float* src = nullptr;
    float* dst = nullptr;
    if (p < total) {
        const int f = (int)(p / F.B);
        const int b = (int)(p - (int64_t)f * F.B);
        const uint32_t x = (uint32_t)((int64_t)ids[p] + (int64_t)F.f_offset[f]);
        const CafeMainBucket* bk = &mb[cafe_hash(x, n1)];
        const uint4 v = *reinterpret_cast<const uint4*>(bk->val);
        const int4 d = *reinterpret_cast<const int4*>(bk->dic);
        int32_t r = 0;
        if (v.w == x && d.w != 0) r = d.w;
        if (v.z == x && d.z != 0) r = d.z;
        if (v.y == x && d.y != 0) r = d.y;
        if (v.x == x && d.x != 0) r = d.x;
        int32_t code;
        if (r) { src = F.w_high + (size_t)(r % F.hotn) * F.D; code = -r; }
        else { const int32_t hr = (int32_t)(x % (uint32_t)F.hash_size[f]); src = F.w_hash[f] + (size_t)hr * F.D; code = hr; }
        const int dr = b / out.rows_per_rank;   // rank that consumes this sample
        dst = out.base[dr] + f * field_stride + (b - dr * out.rows_per_rank) * sample_stride;
        gid_out[p] = x;
        row_out[p] = code;
    }
    constexpr int RPI = 32 / G;   // rows moved per warp iteration
    constexpr int U = 4;
    const int sub = lane / G, c = (lane % G) * 4;
#pragma unroll
    for (int j0 = 0; j0 < 32; j0 += RPI * U) {
        float4 val[U];
        float* d_[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = j0 + u * RPI + sub;
            const float* s = shfl_ptr(src, j);
            d_[u] = shfl_ptr(dst, j);
            if (s) val[u] = ld_row(s + c);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (d_[u]) st_stream(d_[u] + c, val[u]);
    }
}

// The forward in two kernels, for training: k_embed_resolve does the sketch probe only (global id, row code,
// and the two bucket numbers the insert will sort by), k_embed_gather copies the rows named by the codes.
// Between the two the caller can start the backward's sorts, which need nothing but the first kernel's
// outputs, so that they run beside the gather instead of after it.
template <typename IdT>
__global__ void __launch_bounds__(256)
k_embed_resolve(const __grid_constant__ CafeFields F, const IdT* __restrict__ ids, const CafeMainBucket* __restrict__ mb,
                int n1, int n2, uint32_t* __restrict__ gid_out, int32_t* __restrict__ row_out, uint32_t* __restrict__ key1_out,
                uint32_t* __restrict__ key2_out, int total) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    const int f = p / F.B;
    const uint32_t x = (uint32_t)((int64_t)ids[p] + (int64_t)F.f_offset[f]);
    const int32_t k1 = cafe_hash(x, n1);
    const CafeMainBucket* bk = &mb[k1];
    const uint4 v = *reinterpret_cast<const uint4*>(bk->val);
    const int4 d = *reinterpret_cast<const int4*>(bk->dic);
    int32_t r = 0;
    if (v.w == x && d.w != 0) r = d.w;
    if (v.z == x && d.z != 0) r = d.z;
    if (v.y == x && d.y != 0) r = d.y;
    if (v.x == x && d.x != 0) r = d.x;
    gid_out[p] = x;
    row_out[p] = r ? -r : (int32_t)(x % (uint32_t)F.hash_size[f]);
    if (key1_out) { key1_out[p] = (uint32_t)k1; key2_out[p] = (uint32_t)cafe_hash(x, n2); }
}

template <int G>
__global__ void __launch_bounds__(256)
k_embed_gather(const __grid_constant__ CafeFields F, const int32_t* __restrict__ row, const CafeRankBuffers out,
               int64_t field_stride, int64_t sample_stride, int total) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t p = warp * 32 + lane;
    const float* src = nullptr;
    float* dst = nullptr;
    if (p < total) {
        const int f = (int)(p / F.B);
        const int b = (int)(p - (int64_t)f * F.B);
        const int32_t code = row[p];
        src = code < 0 ? F.w_high + (size_t)((-code) % F.hotn) * F.D : F.w_hash[f] + (size_t)code * F.D;
        const int dr = b / out.rows_per_rank;   // rank that consumes this sample
        dst = out.base[dr] + f * field_stride + (b - dr * out.rows_per_rank) * sample_stride;
    }
    constexpr int RPI = 32 / G;   // rows moved per warp iteration
    constexpr int U = 4;
    const int sub = lane / G, c = (lane % G) * 4;
#pragma unroll
    for (int j0 = 0; j0 < 32; j0 += RPI * U) {
        float4 val[U];
        float* d_[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = j0 + u * RPI + sub;
            const float* s = shfl_ptr(src, j);
            d_[u] = shfl_ptr(dst, j);
            if (s) val[u] = ld_row(s + c);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (d_[u]) st_stream(d_[u] + c, val[u]);
    }
}

// ---------------------------------------------------------------------------------------------
// importance (sk_embedding_bag.py:178-189): per-lookup L2 norm of its gradient row, scaled by
// N / (sum of the field's norms).
// ---------------------------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(256)
k_grad_norm(const float* __restrict__ grad, int64_t field_stride, int64_t sample_stride, int B, int total,
            float* __restrict__ norm) {
    // a group of G lanes takes 4 consecutive lookups: 4 independent 16-byte loads per lane in flight
    constexpr int U = 4;
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t p0 = (t / G) * U;
    const int c = (int)(t % G) * 4;
    float s[U];
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t p = p0 + u;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p < total) {
            const int f = (int)(p / B);
            const int b = (int)(p - (int64_t)f * B);
            v[u] = ld_stream(grad + f * field_stride + b * sample_stride + c);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        s[u] = v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) s[u] += __shfl_xor_sync(FULL, s[u], o);
    }
    if (c == 0) {
#pragma unroll
        for (int u = 0; u < U; ++u) if (p0 + u < total) norm[p0 + u] = sqrtf(s[u]);
    }
}

// one block per field: fixed-order sum of the field's norms
__global__ void __launch_bounds__(1024) k_field_sum(const float* __restrict__ norm, int B, float* __restrict__ totals) {
    __shared__ float sh[1024];
    const float* x = norm + (size_t)blockIdx.x * B;
    float s = 0.f;
    for (int i = threadIdx.x; i < B; i += 1024) s += x[i];
    sh[threadIdx.x] = s;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = sh[0];
}

__global__ void k_importance(const float* __restrict__ norm, const float* __restrict__ totals, int B, int total,
                             float* __restrict__ imp) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    const float tot = totals[p / B];
    // a field whose whole gradient is zero would give 0/0 in the reference; counts stay unchanged here
    imp[p] = tot > 0.f ? __fdiv_rn(__fmul_rn(norm[p], (float)B), tot) : 0.f;
}

// ---------------------------------------------------------------------------------------------
// migration (sk_embedding_bag.py:205-208, guarded): a lookup that was handed a hot row and whose id
// is in the main table right after its field's call gets its hash row copied into that hot row.
// The hash row is addressed with the LOCAL id, as the reference does at :207.
// ---------------------------------------------------------------------------------------------
// Two lookups of one call can name the same hot row: an id of an early field is handed row r, a threshold
// re-fit at a later field's call boundary takes r away again, and an id of that later field pops r.  The
// reference migrates field by field, so the later copy is the one that stays.  Here all fields migrate in
// one launch, so the lookups first claim their row (the highest position wins, k_migrate_claim) and only
// the winner copies; it also returns the claim slot to -1 for the next call.
__global__ void __launch_bounds__(256)
k_migrate_claim(const int32_t* __restrict__ mask, const int32_t* __restrict__ post_row, int total, int32_t* __restrict__ winner) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p < total && mask[p] != 0 && post_row[p] > 0) atomicMax(&winner[post_row[p]], p);
}
template <typename IdT>
__global__ void __launch_bounds__(256)
k_migrate(const __grid_constant__ CafeFields F, const IdT* __restrict__ ids, const int32_t* __restrict__ mask,
          const int32_t* __restrict__ post_row, int total, int32_t* __restrict__ winner, int32_t* __restrict__ n_migrated) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t p = warp * 32 + lane;
    const float* src = nullptr;
    float* dst = nullptr;
    if (p < total && mask[p] != 0 && post_row[p] > 0 && winner[post_row[p]] == (int32_t)p) {
        const int f = (int)(p / F.B);
        const int64_t local = (int64_t)ids[p];
        src = F.w_hash[f] + (size_t)(local % F.hash_size[f]) * F.D;
        dst = F.w_high + (size_t)post_row[p] * F.D;
        winner[post_row[p]] = -1;
    }
    unsigned act = __ballot_sync(FULL, dst != nullptr);
    if (lane == 0 && act && n_migrated) atomicAdd(n_migrated, __popc(act));
    while (act) {
        const int j = __ffs(act) - 1;
        act &= act - 1;
        const float* s = shfl_ptr(src, j);
        float* d = shfl_ptr(dst, j);
        for (int c = lane * 4; c < F.D; c += 128) *reinterpret_cast<float4*>(d + c) = *reinterpret_cast<const float4*>(s + c);
    }
}

// ---------------------------------------------------------------------------------------------
// scatter + SGD.  Lookups are sorted by unified row (hot rows first, then each field's hash rows);
// a group of G lanes reduces a chunk of CAFE_CHUNK consecutive sorted lookups in order.  Rows whose
// lookups lie inside one chunk are updated at once; rows that span chunks leave per-chunk partial
// sums that a second kernel adds in chunk order.  The order of additions is fixed by the sort, so
// results are deterministic.
// ---------------------------------------------------------------------------------------------
__global__ void k_row_keys(const __grid_constant__ CafeFields F, const int32_t* __restrict__ row, int total,
                           uint32_t* __restrict__ key) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    const int32_t r = row[p];
    key[p] = r < 0 ? (uint32_t)((-r) % F.hotn) : (uint32_t)(F.hotn + F.hash_base[p / F.B] + r);
}

__device__ __forceinline__ float* row_ptr(const CafeFields& F, uint32_t key, int pos) {
    if (key < (uint32_t)F.hotn) return F.w_high + (size_t)key * F.D;
    const int f = pos / F.B;
    return F.w_hash[f] + (size_t)(key - (uint32_t)F.hotn - (uint32_t)F.hash_base[f]) * F.D;
}
// row -= lr * g.  Every row is updated exactly once per call (by the chunk that holds all of its
// lookups, or by the fix-up pass), so the update can be a fire-and-forget vector reduction at L2
// instead of a load / subtract / store round trip; with a single add per element the result does
// not depend on timing.
__device__ __forceinline__ void sgd_apply(float* w, float4 g, float lr) {
    atomicAdd(reinterpret_cast<float4*>(w), make_float4(-(lr * g.x), -(lr * g.y), -(lr * g.z), -(lr * g.w)));
}

#define NOKEY 0xffffffffu

template <int G>
__global__ void __launch_bounds__(256, 4)
k_scatter_chunks(const __grid_constant__ CafeFields F, const float* __restrict__ grad, int64_t field_stride,
                 int64_t sample_stride, const uint32_t* __restrict__ skey, const int32_t* __restrict__ spos, int M,
                 float lr, float* __restrict__ partial) {
    constexpr int PER = CAFE_CHUNK / G;   // sorted entries held per lane
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t chunk = t / G;
    const int gl = (int)(t % G);          // lane within the group
    const int c = gl * 4;
    const int64_t base = chunk * CAFE_CHUNK;
    const int cnt = (int)max((int64_t)0, min((int64_t)CAFE_CHUNK, (int64_t)M - base));
    uint32_t k[PER];
    int32_t q[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int j = i * G + gl;
        k[i] = j < cnt ? skey[base + j] : NOKEY;
        q[i] = j < cnt ? spos[base + j] : 0;
    }
    const uint32_t key_prev = (cnt > 0 && base > 0) ? skey[base - 1] : NOKEY;
    const uint32_t key_next = (cnt > 0 && base + CAFE_CHUNK < M) ? skey[base + CAFE_CHUNK] : NOKEY;

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t cur = NOKEY;
    int cur_pos = 0;
    bool first_seg = true;
    const int B = F.B;
    constexpr int U = 8;
#pragma unroll
    for (int j0 = 0; j0 < CAFE_CHUNK; j0 += U) {
        float4 v[U];
        uint32_t kk[U];
        int32_t qq[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = j0 + u;
            kk[u] = __shfl_sync(FULL, k[j / G], j % G, G);
            qq[u] = __shfl_sync(FULL, q[j / G], j % G, G);
            if (kk[u] != NOKEY) {
                const int f = qq[u] / B;
                const int b = qq[u] - f * B;
                v[u] = ld_stream(grad + f * field_stride + b * sample_stride + c);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (kk[u] == NOKEY) continue;
            if (kk[u] != cur) {
                if (cur != NOKEY) {
                    // a row that ended inside the chunk: complete unless it came in from the previous chunk
                    if (first_seg && cur == key_prev) *reinterpret_cast<float4*>(partial + (size_t)(chunk * 2) * CAFE_MAX_DIM + c) = acc;
                    else sgd_apply(row_ptr(F, cur, cur_pos) + c, acc, lr);
                    first_seg = false;
                }
                cur = kk[u];
                cur_pos = qq[u];
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
        }
    }
    if (cur != NOKEY) {
        const bool open_left = first_seg && cur == key_prev;
        const bool open_right = cur == key_next;
        if (open_left || open_right)
            *reinterpret_cast<float4*>(partial + (size_t)(chunk * 2 + (first_seg ? 0 : 1)) * CAFE_MAX_DIM + c) = acc;
        else
            sgd_apply(row_ptr(F, cur, cur_pos) + c, acc, lr);
    }
}

// One group per chunk; the chunk in which a spanning row STARTS adds up that row's partial sums.
template <int G>
__global__ void __launch_bounds__(256)
k_scatter_fixup(const __grid_constant__ CafeFields F, const uint32_t* __restrict__ skey,
                const int32_t* __restrict__ spos, int M, float lr, const float* __restrict__ partial) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t chunk = t / G;
    const int c = (int)(t % G) * 4;
    const int64_t base = chunk * CAFE_CHUNK;
    if (base + CAFE_CHUNK >= M) return;   // the last chunk cannot continue to the right
    const uint32_t key = skey[base + CAFE_CHUNK - 1];
    if (key != skey[base + CAFE_CHUNK]) return;            // its last row ends with the chunk
    const bool single = skey[base] == key;
    if (single && base > 0 && skey[base - 1] == key) return;   // the row started in an earlier chunk
    // end of the row's range in the sorted keys
    int64_t lo = base + CAFE_CHUNK, hi = M;   // first index with key' > key lies in (lo, hi]
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (skey[mid] <= key) lo = mid + 1; else hi = mid;
    }
    const int64_t last_chunk = (lo - 1) / CAFE_CHUNK;
    float4 acc = *reinterpret_cast<const float4*>(partial + (size_t)(chunk * 2 + (single ? 0 : 1)) * CAFE_MAX_DIM + c);
    constexpr int U = 8;
    for (int64_t c0 = chunk + 1; c0 <= last_chunk; c0 += U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c0 + u <= last_chunk) v[u] = *reinterpret_cast<const float4*>(partial + (size_t)((c0 + u) * 2) * CAFE_MAX_DIM + c);
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c0 + u <= last_chunk) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    sgd_apply(row_ptr(F, key, spos[base + CAFE_CHUNK - 1]) + c, acc, lr);
}

// ---------------------------------------------------------------------------------------------
// Field-sharded exchange over peer memory (NVLink): no counterpart in the reference, which is
// single-GPU.  Every rank owns the fields f with f % nranks == rank and serves them for the global
// batch; buffers of other ranks are plain peer mappings (ordinary loads and stores, no multicast).
//   ids      : each rank stores its batch slice of every field's ids straight into the owners' id
//              buffers ([F_owner, nranks * rows] per owner);
//   forward  : the gather kernel above stores each pooled row into the buffer of the rank that
//              consumes the sample (CafeRankBuffers), i.e. the all-to-all is the kernel's epilogue;
//   backward : the owner pulls the gradient rows of its fields from the consumers' buffers while it
//              computes their norms, keeping a local copy for the scatter (all-to-all as prologue).
// Ordering between ranks (data ready / buffer free) is the caller's: a stream-ordered collective
// between the phases.
// ---------------------------------------------------------------------------------------------
struct CafeIdBuffers {
    int64_t* base[CAFE_MAX_RANKS];
};
__global__ void k_scatter_ids(const int64_t* __restrict__ ids, int nfields, int rows, int nranks, int rank,
                              const CafeIdBuffers dst) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (int64_t)nfields * rows) return;
    const int f = (int)(t / rows), b = (int)(t - (int64_t)f * rows);
    const int owner = f % nranks, j = f / nranks;   // j = index of f among its owner's fields
    dst.base[owner][(int64_t)j * nranks * rows + (int64_t)rank * rows + b] = ids[t];
}

// Consumer side of the gradient exchange: this rank's gradient buffer holds, per owner g, a block
// [rows, F_g, D]; every row is stored into owner g's buffer at sample (rank*rows + b) -- remote
// stores, which NVLink handles better than remote loads.
struct CafePushPlan {
    float* base[CAFE_MAX_RANKS];       // owner g's gradient buffer [nranks*rows, F_g, D]
    int32_t fields_of[CAFE_MAX_RANKS];  // F_g
    int32_t row_off[CAFE_MAX_RANKS + 1];   // first (sample, field) row of owner g's block in this rank's buffer
};
__global__ void __launch_bounds__(256)
k_push_grads(const float* __restrict__ grad, const CafePushPlan P, int nranks, int rank, int rows, int D, int64_t total_rows,
             int j_begin, int j_end) {
    const int lanes = D / 4;                       // lanes per row (16-byte vectors)
    // A grid of a few blocks per SM walks the rows: the transfer is bound by NVLink, not by the number of threads in
    // flight, and a launch that filled every SM would hold back the small kernels of the sketch insert that run
    // beside it on another stream.
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total_rows * lanes; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t q0 = t / lanes;
        const int c = (int)(t % lanes) * 4;
        // Every rank starts with the block of the owner after itself and goes round: at any moment the ranks
        // store into different owners, so no owner's NVLink ingress has to take all of them at once.
        int64_t q = q0 + P.row_off[(rank + 1) % nranks];
        if (q >= total_rows) q -= total_rows;
        int g = 0;
        while (g + 1 < nranks && q >= P.row_off[g + 1]) ++g;
        const int64_t local = q - P.row_off[g];        // row inside block g: b * F_g + j
        const int fg = P.fields_of[g];
        const int64_t b = local / fg, j = local - b * fg;
        if (j < j_begin || j >= j_end) continue;   // only the owners' fields number j_begin .. j_end-1 go in this launch
        const float4 v = ld_stream(grad + q * D + c);
        *reinterpret_cast<float4*>(P.base[g] + (((int64_t)rank * rows + b) * fg + j) * D + c) = v;
    }
}

// The norms of the same rows, sent ahead of them: the sketch insert needs only the per-lookup L2 norms, which are a
// 128th of the rows' bytes, so the owners can start inserting while the rows themselves are still crossing NVLink.
// Arithmetic and lane layout are those of k_grad_norm (which the owner would run on the delivered rows): a group of G
// lanes squares and adds the same 16-byte pieces in the same butterfly, so the owner gets the bits it would compute.
// Owner g's norm array is [F_g, nranks*rows] (field-major, as k_field_sum and k_importance read it).  The norms are
// first written to a local staging array in the order they will have at the owners (per owner g a block [F_g, rows]);
// k_send_norms then copies every block's field rows with consecutive lanes on consecutive floats, so the remote
// stores leave as full 128-byte lines instead of one 4-byte store per lookup.
template <int G>
__global__ void __launch_bounds__(256)
k_push_norms(const float* __restrict__ grad, const CafePushPlan P, int nranks, int rows, int64_t total_rows,
             float* __restrict__ staged) {
    constexpr int U = 4;
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q0 = (t / G) * U;
    const int c = (int)(t % G) * 4;
    float s[U];
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + u < total_rows) v[u] = ld_stream(grad + (q0 + u) * (int64_t)(G * 4) + c);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        s[u] = v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) s[u] += __shfl_xor_sync(FULL, s[u], o);
    }
    if (c == 0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t q = q0 + u;
            if (q >= total_rows) break;
            int g = 0;
            while (g + 1 < nranks && q >= P.row_off[g + 1]) ++g;
            const int64_t local = q - P.row_off[g];        // row inside block g: b * F_g + j
            const int fg = P.fields_of[g];
            const int64_t b = local / fg, j = local - b * fg;
            staged[P.row_off[g] + j * rows + b] = sqrtf(s[u]);
        }
    }
}
__global__ void __launch_bounds__(256)
k_send_norms(const float* __restrict__ staged, const CafePushPlan P, int nranks, int rank, int rows, int64_t total_rows) {
    const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= total_rows) return;
    int g = 0;
    while (g + 1 < nranks && q >= P.row_off[g + 1]) ++g;
    const int64_t local = q - P.row_off[g];        // inside block g: j * rows + b
    const int64_t j = local / rows, b = local - j * rows;
    P.base[g][j * ((int64_t)nranks * rows) + (int64_t)rank * rows + b] = staged[q];
}

template <int G>
__global__ void __launch_bounds__(256)
k_pull_norm(const CafeRankBuffers src, int64_t field_stride, int64_t sample_stride, int B, int total,
            float* __restrict__ local, float* __restrict__ norm) {
    constexpr int U = 4;
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t p0 = (t / G) * U;
    const int c = (int)(t % G) * 4;
    float s[U];
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t p = p0 + u;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p < total) {
            const int f = (int)(p / B);
            const int b = (int)(p - (int64_t)f * B);
            const int r = b / src.rows_per_rank;
            v[u] = *reinterpret_cast<const float4*>(src.base[r] + f * field_stride + (b - r * src.rows_per_rank) * sample_stride + c);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t p = p0 + u;
        if (p < total) {
            const int f = (int)(p / B);
            const int b = (int)(p - (int64_t)f * B);
            *reinterpret_cast<float4*>(local + f * field_stride + b * sample_stride + c) = v[u];
        }
        s[u] = v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) s[u] += __shfl_xor_sync(FULL, s[u], o);
    }
    if (c == 0) {
#pragma unroll
        for (int u = 0; u < U; ++u) if (p0 + u < total) norm[p0 + u] = sqrtf(s[u]);
    }
}

// ---------------------------------------------------------------------------------------------
// Input records -> batch.  The reference's preprocessed datasets store the categorical features sample-major
// (processed_sparse_sep.bin: int32 [N, F], ArtifactEvaluation/load_data.py:44-66; the same layout for the Kaggle
// / Terabyte / Avazu memmaps of dlrm_data_pytorch.py:643-649) and its collate functions turn a block of rows into
// one int64 index vector per field on the host (dlrm_data_pytorch.py:395-437: X_cat[:, i] for every field, labels
// as float [B, 1]).  Here the block of rows is copied to the device as it lies on disk and transposed there:
// a 32 x 32 tile goes through shared memory so that both the reads (along a sample's fields) and the writes
// (along a field's samples) are coalesced.
// ---------------------------------------------------------------------------------------------
template <typename OutT>
__global__ void __launch_bounds__(256) k_records_to_fields(const int32_t* __restrict__ rows, int B, int F, OutT* __restrict__ ids) {
    __shared__ int32_t tile[32][33];
    const int b0 = blockIdx.x * 32, f0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8 threads
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int b = b0 + r, f = f0 + tx;
        if (b < B && f < F) tile[r][tx] = rows[(int64_t)b * F + f];
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int f = f0 + r, b = b0 + tx;
        if (b < B && f < F) ids[(int64_t)f * B + b] = (OutT)tile[tx][r];
    }
}
__global__ void k_labels_to_float(const int32_t* __restrict__ label, int B, float* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) out[i] = (float)label[i];
}

// ---------------------------------------------------------------------------------------------
// workspace
// ---------------------------------------------------------------------------------------------
int cafe_embed_ws_init(CafeEmbedWorkspace* ws, int cap, int hotn) {
    ws->cap = cap;
    const size_t M = (size_t)cap;
    const size_t chunks = (M + CAFE_CHUNK - 1) / CAFE_CHUNK;
    cudaError_t e = cudaSuccess;
    auto A = [&](void** p, size_t n) { if (e == cudaSuccess) e = cudaMalloc(p, n ? n : 1); };
    A((void**)&ws->norm, 4 * M); A((void**)&ws->imp, 4 * M); A((void**)&ws->totals, 4 * CAFE_MAX_SEGMENTS);
    A((void**)&ws->mask, 4 * M); A((void**)&ws->post_row, 4 * M);
    for (int i = 0; i < 2; ++i) { A((void**)&ws->key[i], 4 * M); A((void**)&ws->pos[i], 4 * M); }
    A((void**)&ws->partial, sizeof(float) * 2 * chunks * CAFE_MAX_DIM);
    A((void**)&ws->row_winner, 4 * (size_t)(hotn > 0 ? hotn : 1));
    if (e == cudaSuccess) e = cudaMemset(ws->row_winner, 0xff, 4 * (size_t)(hotn > 0 ? hotn : 1));   // -1: unclaimed
    A((void**)&ws->key_tmp, 4 * M);
    A((void**)&ws->bucket_key[0], 4 * M); A((void**)&ws->bucket_key[1], 4 * M);
    A((void**)&ws->sort_scratch, 4 * cafe_rs_scratch_elems(cap));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ws->side, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ws->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ws->ev_join, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ws->late, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ws->ev_late, cudaEventDisableTiming);
    if (e != cudaSuccess) { cafe_internal_set_error(cudaGetErrorString(e)); return CAFE_ERR_CUDA; }
    return CAFE_OK;
}

void cafe_embed_ws_free(CafeEmbedWorkspace* ws) {
    void* ptrs[] = {ws->norm, ws->imp, ws->totals, ws->mask, ws->post_row, ws->key[0], ws->key[1], ws->pos[0], ws->pos[1],
                    ws->partial, ws->key_tmp, ws->sort_scratch, ws->row_winner, ws->bucket_key[0], ws->bucket_key[1]};
    for (void* p : ptrs) if (p) cudaFree(p);
    if (ws->side) { cudaStreamSynchronize(ws->side); cudaStreamDestroy(ws->side); }
    if (ws->ev_fork) cudaEventDestroy(ws->ev_fork);
    if (ws->ev_join) cudaEventDestroy(ws->ev_join);
    if (ws->late) { cudaStreamSynchronize(ws->late); cudaStreamDestroy(ws->late); }
    if (ws->ev_late) cudaEventDestroy(ws->ev_late);
    *ws = CafeEmbedWorkspace();
}

// ---------------------------------------------------------------------------------------------
// C ABI (embedding part)
// ---------------------------------------------------------------------------------------------
static int fail_cuda(const char* where) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return CAFE_OK;
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: %s", where, cudaGetErrorString(e));
    cafe_internal_set_error(buf);
    return CAFE_ERR_CUDA;
}
static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

static int fill_fields(CafeFields* F, int nfields, int B, int D, int hotn, const int64_t* f_offset, const int32_t* hash_size,
                       float* const* w_hash, float* w_high) {
    if (nfields < 1 || nfields > CAFE_MAX_SEGMENTS || B < 0 || hotn < 1 || !f_offset || !hash_size || !w_hash || !w_high)
        return CAFE_ERR_ARG;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    if ((int64_t)nfields * B > 0x7fffffffLL) return CAFE_ERR_CAPACITY;
    memset(F, 0, sizeof(*F));
    F->nfields = nfields; F->B = B; F->D = D; F->hotn = hotn; F->w_high = w_high;
    if (!aligned16(w_high)) return CAFE_ERR_ARG;
    int64_t base = 0;
    for (int f = 0; f < nfields; ++f) {
        if (hash_size[f] < 1 || !w_hash[f] || !aligned16(w_hash[f])) return CAFE_ERR_ARG;
        F->f_offset[f] = (uint32_t)f_offset[f];
        F->hash_size[f] = hash_size[f];
        F->hash_base[f] = (int32_t)base;
        F->w_hash[f] = w_hash[f];
        base += hash_size[f];
        if (base + hotn > 0x7fffffffLL) return CAFE_ERR_CAPACITY;
    }
    F->hash_base[nfields] = (int32_t)base;
    return CAFE_OK;
}

static bool strides_ok(const float* p, int64_t fs, int64_t ss) { return aligned16(p) && fs % 4 == 0 && ss % 4 == 0; }

#define DISPATCH_G(D, CALL)              \
    switch ((D) / 4) {                   \
        case 4: { constexpr int G = 4; CALL; } break;   \
        case 8: { constexpr int G = 8; CALL; } break;   \
        case 16: { constexpr int G = 16; CALL; } break; \
        default: { constexpr int G = 32; CALL; } break; \
    }

static int launch_forward(const CafeFields& F, const void* ids_dev, int ids_are_int64, const CafeSketchView& V,
                          const CafeRankBuffers& out_dev, int64_t out_field_stride, int64_t out_sample_stride,
                          uint32_t* gid_out_dev, int32_t* row_out_dev, int total, int D, cudaStream_t st) {
    const int warps = (total + 31) / 32;
    const int blocks = (warps + 7) / 8;
    CAFE_PROF(CAFE_P_FORWARD, st);
    if (ids_are_int64) {
        DISPATCH_G(D, (k_embed_forward<G, int64_t><<<blocks, 256, 0, st>>>(F, (const int64_t*)ids_dev, V.main, V.n1, out_dev,
                       out_field_stride, out_sample_stride, gid_out_dev, row_out_dev, total)));
    } else {
        DISPATCH_G(D, (k_embed_forward<G, int32_t><<<blocks, 256, 0, st>>>(F, (const int32_t*)ids_dev, V.main, V.n1, out_dev,
                       out_field_stride, out_sample_stride, gid_out_dev, row_out_dev, total)));
    }
    return fail_cuda("cafe_embed_forward");
}

extern "C" {

int cafe_embed_forward(void* h, const void* ids_dev, int ids_are_int64, int nfields, int B, const int64_t* f_offset,
                       const int32_t* hash_size, float* const* weight_hash, float* weight_high, int hotn, int D,
                       float* out_dev, int64_t out_field_stride, int64_t out_sample_stride, uint32_t* gid_out_dev,
                       int32_t* row_out_dev, void* stream) {
    if (!h) return CAFE_ERR_ARG;
    CafeFields F;
    int rc = fill_fields(&F, nfields, B, D, hotn, f_offset, hash_size, weight_hash, weight_high);
    if (rc != CAFE_OK) return rc;
    const int total = nfields * B;
    if (total == 0) return CAFE_OK;
    if (!ids_dev || !out_dev || !gid_out_dev || !row_out_dev || !strides_ok(out_dev, out_field_stride, out_sample_stride))
        return CAFE_ERR_ARG;
    CafeSketchView V = cafe_internal_view(h);
    if (hotn != V.lim) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    CafeRankBuffers ob;
    memset(&ob, 0, sizeof(ob));
    ob.base[0] = out_dev;
    ob.rows_per_rank = B > 0 ? B : 1;
    return launch_forward(F, ids_dev, ids_are_int64, V, ob, out_field_stride, out_sample_stride, gid_out_dev, row_out_dev, total, D, st);
}


int cafe_records_to_batch(const int32_t* sparse_rows_dev, int B, int F, void* ids_out_dev, int ids_are_int64,
                          const int32_t* label_dev, float* label_out_dev, void* stream) {
    if (B < 0 || F < 1) return CAFE_ERR_ARG;
    if (B == 0) return CAFE_OK;
    if (!sparse_rows_dev || !ids_out_dev) return CAFE_ERR_ARG;
    if ((label_dev == nullptr) != (label_out_dev == nullptr)) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    CAFE_PROF(CAFE_P_OTHER, st);
    const dim3 grid((unsigned)((B + 31) / 32), (unsigned)((F + 31) / 32));
    if (ids_are_int64) k_records_to_fields<int64_t><<<grid, 256, 0, st>>>(sparse_rows_dev, B, F, (int64_t*)ids_out_dev);
    else k_records_to_fields<int32_t><<<grid, 256, 0, st>>>(sparse_rows_dev, B, F, (int32_t*)ids_out_dev);
    if (label_dev) k_labels_to_float<<<(B + 255) / 256, 256, 0, st>>>(label_dev, B, label_out_dev);
    return fail_cuda("cafe_records_to_batch");
}

int cafe_embed_resolve(void* h, const void* ids_dev, int ids_are_int64, int nfields, int B, const int64_t* f_offset,
                       const int32_t* hash_size, int hotn, uint32_t* gid_out_dev, int32_t* row_out_dev, void* stream) {
    if (!h || nfields < 1 || nfields > CAFE_MAX_SEGMENTS || B < 0 || !f_offset || !hash_size) return CAFE_ERR_ARG;
    const int64_t total64 = (int64_t)nfields * B;
    if (total64 > 0x7fffffffLL) return CAFE_ERR_CAPACITY;
    if (total64 == 0) return CAFE_OK;
    if (!ids_dev || !gid_out_dev || !row_out_dev) return CAFE_ERR_ARG;
    CafeFields F;
    memset(&F, 0, sizeof(F));
    F.nfields = nfields; F.B = B; F.hotn = hotn;
    for (int f = 0; f < nfields; ++f) {
        if (hash_size[f] < 1) return CAFE_ERR_ARG;
        F.f_offset[f] = (uint32_t)f_offset[f]; F.hash_size[f] = hash_size[f];
    }
    CafeSketchView V = cafe_internal_view(h);
    if (hotn != V.lim) return CAFE_ERR_ARG;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    const int total = (int)total64;
    // the bucket numbers are kept for the insert's sorts when the lookups fit the workspace
    const bool keep = total <= ws->cap;
    uint32_t* k1 = keep ? ws->bucket_key[0] : nullptr;
    uint32_t* k2 = keep ? ws->bucket_key[1] : nullptr;
    ws->keys_of = keep ? gid_out_dev : nullptr;
    ws->keys_total = keep ? total : 0;
    cudaStream_t st = (cudaStream_t)stream;
    CAFE_PROF(CAFE_P_QUERY, st);
    const int blocks = (total + 255) / 256;
    if (ids_are_int64) k_embed_resolve<int64_t><<<blocks, 256, 0, st>>>(F, (const int64_t*)ids_dev, V.main, V.n1, V.n2, gid_out_dev, row_out_dev, k1, k2, total);
    else k_embed_resolve<int32_t><<<blocks, 256, 0, st>>>(F, (const int32_t*)ids_dev, V.main, V.n1, V.n2, gid_out_dev, row_out_dev, k1, k2, total);
    return fail_cuda("cafe_embed_resolve");
}

static int gather_impl(void* h, const int32_t* row_dev, int nfields, int B, const int32_t* hash_size, float* const* weight_hash,
                       float* weight_high, int hotn, int D, const CafeRankBuffers& ob, int64_t out_field_stride,
                       int64_t out_sample_stride, cudaStream_t st) {
    CafeFields F;
    int64_t zero_off[CAFE_MAX_SEGMENTS] = {0};
    int rc = fill_fields(&F, nfields, B, D, hotn, zero_off, hash_size, weight_hash, weight_high);
    if (rc != CAFE_OK) return rc;
    const int total = nfields * B;
    if (total == 0) return CAFE_OK;
    if (!h || !row_dev || out_field_stride % 4 || out_sample_stride % 4) return CAFE_ERR_ARG;
    const int warps = (total + 31) / 32;
    const int blocks = (warps + 7) / 8;
    CAFE_PROF(CAFE_P_FORWARD, st);
    DISPATCH_G(D, (k_embed_gather<G><<<blocks, 256, 0, st>>>(F, row_dev, ob, out_field_stride, out_sample_stride, total)));
    return fail_cuda("cafe_embed_gather");
}

int cafe_embed_gather(void* h, const int32_t* row_dev, int nfields, int B, const int32_t* hash_size, float* const* weight_hash,
                      float* weight_high, int hotn, int D, float* out_dev, int64_t out_field_stride, int64_t out_sample_stride,
                      void* stream) {
    if (nfields * (int64_t)B > 0 && (!out_dev || !aligned16(out_dev))) return CAFE_ERR_ARG;
    CafeRankBuffers ob;
    memset(&ob, 0, sizeof(ob));
    ob.base[0] = out_dev;
    ob.rows_per_rank = B > 0 ? B : 1;
    return gather_impl(h, row_dev, nfields, B, hash_size, weight_hash, weight_high, hotn, D, ob, out_field_stride, out_sample_stride,
                       (cudaStream_t)stream);
}

int cafe_embed_gather_sharded(void* h, const int32_t* row_dev, int nfields, int B, const int32_t* hash_size,
                              float* const* weight_hash, float* weight_high, int hotn, int D, float* const* out_rank, int nranks,
                              int rows_per_rank, int64_t out_field_stride, int64_t out_sample_stride, void* stream) {
    if (!out_rank || nranks < 1 || nranks > CAFE_MAX_RANKS || rows_per_rank < 1) return CAFE_ERR_ARG;
    if ((int64_t)rows_per_rank * nranks != B) return CAFE_ERR_ARG;
    CafeRankBuffers ob;
    memset(&ob, 0, sizeof(ob));
    for (int r = 0; r < nranks; ++r) { if (!out_rank[r] || !aligned16(out_rank[r])) return CAFE_ERR_ARG; ob.base[r] = out_rank[r]; }
    ob.rows_per_rank = rows_per_rank;
    return gather_impl(h, row_dev, nfields, B, hash_size, weight_hash, weight_high, hotn, D, ob, out_field_stride, out_sample_stride,
                       (cudaStream_t)stream);
}

int cafe_grad_importance(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride, int nfields, int B,
                         int D, float* imp_out_dev, void* stream) {
    if (!h || nfields < 1 || nfields > CAFE_MAX_SEGMENTS || B < 0) return CAFE_ERR_ARG;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    const int64_t total64 = (int64_t)nfields * B;
    if (total64 == 0) return CAFE_OK;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    if (total64 > ws->cap) return CAFE_ERR_CAPACITY;
    if (!grad_dev || !imp_out_dev || !strides_ok(grad_dev, field_stride, sample_stride)) return CAFE_ERR_ARG;
    const int total = (int)total64;
    cudaStream_t st = (cudaStream_t)stream;
    { CAFE_PROF(CAFE_P_NORM, st);
    DISPATCH_G(D, (k_grad_norm<G><<<(unsigned)((((int64_t)total + 3) / 4 * G + 255) / 256), 256, 0, st>>>(grad_dev, field_stride,
                   sample_stride, B, total, ws->norm))); }
    { CAFE_PROF(CAFE_P_FIELDSUM, st); k_field_sum<<<nfields, 1024, 0, st>>>(ws->norm, B, ws->totals); }
    { CAFE_PROF(CAFE_P_IMPORTANCE, st); k_importance<<<(total + 255) / 256, 256, 0, st>>>(ws->norm, ws->totals, B, total, imp_out_dev); }
    return fail_cuda("cafe_grad_importance");
}

// ---------------------------------------------------------------------------------------------
// Importance without any allocation.
//
// cafe_grad_importance keeps its two intermediates (one norm per lookup, one sum per field) in a
// workspace that cafe_sketch_create obtained with cudaMalloc.  Some hosts cannot do that: a serving
// process that handed the whole device to its own memory pool at start-up and forbids further
// allocation, or a caller that must not take the device-wide stall an allocation can cause in the
// middle of its step.  For them the same three kernels run here on a scratch area that is part of
// the library image: a file-scope __device__ array, which every GPU that loads the library holds
// from load to exit (CAFE_STATIC_IMPORTANCE_MAX floats for the norms plus one float per field,
// about 1 MiB).  No handle is needed, and nothing is allocated or freed here: not with the CUDA
// runtime, not through any library.
//
// The array's name is a host-side stand-in in host code, not a device address, so the address the
// kernels get is looked up with cudaGetSymbolAddress -- once per device, on the first call made
// while that device is current.  That first call should therefore come before any stream capture.
// Every call on a device shares the one array: calls that can overlap on the GPU (different
// streams, different host threads) race on it; run them one after the other.  Nothing in the array
// has to start at zero -- each call writes every element before it reads it -- so it is not
// cleared between calls.
// ---------------------------------------------------------------------------------------------
#define CAFE_STATIC_IMPORTANCE_MAX (1 << 18)   // most lookups (nfields * B) one call may cover
#define CAFE_STATIC_MAX_DEVICES 64
static __device__ __align__(256) float g_static_importance_scratch[CAFE_STATIC_IMPORTANCE_MAX + CAFE_MAX_SEGMENTS];
static float* g_static_scratch_addr[CAFE_STATIC_MAX_DEVICES];   // per device, filled on first use

int cafe_grad_importance_static(const float* grad_dev, int64_t field_stride, int64_t sample_stride, int nfields, int B,
                                int D, float* imp_out_dev, void* stream) {
    if (nfields < 1 || nfields > CAFE_MAX_SEGMENTS || B < 0) return CAFE_ERR_ARG;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    const int64_t total64 = (int64_t)nfields * B;
    if (total64 > CAFE_STATIC_IMPORTANCE_MAX) {
        char buf[160];
        snprintf(buf, sizeof(buf), "cafe_grad_importance_static: %lld lookups exceed the built-in scratch of %d",
                 (long long)total64, CAFE_STATIC_IMPORTANCE_MAX);
        cafe_internal_set_error(buf);
        return CAFE_ERR_CAPACITY;
    }
    if (total64 == 0) return CAFE_OK;
    if (!grad_dev || !imp_out_dev || !strides_ok(grad_dev, field_stride, sample_stride)) return CAFE_ERR_ARG;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= CAFE_STATIC_MAX_DEVICES) {
        cafe_internal_set_error(e != cudaSuccess ? cudaGetErrorString(e) : "cafe_grad_importance_static: device index out of range");
        return e != cudaSuccess ? CAFE_ERR_CUDA : CAFE_ERR_UNSUPPORTED;
    }
    float* scratch = g_static_scratch_addr[dev];
    if (!scratch) {   // set-up, once per device, with that device current
        e = cudaGetSymbolAddress((void**)&scratch, g_static_importance_scratch);
        if (e != cudaSuccess || !scratch) {
            cafe_internal_set_error(e != cudaSuccess ? cudaGetErrorString(e) : "cafe_grad_importance_static: no symbol address");
            return CAFE_ERR_CUDA;
        }
        g_static_scratch_addr[dev] = scratch;
    }
    float* norm = scratch;                                   // [total]
    float* totals = scratch + CAFE_STATIC_IMPORTANCE_MAX;    // [nfields]
    const int total = (int)total64;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH_G(D, (k_grad_norm<G><<<(unsigned)((((int64_t)total + 3) / 4 * G + 255) / 256), 256, 0, st>>>(grad_dev, field_stride,
                   sample_stride, B, total, norm)));
    k_field_sum<<<nfields, 1024, 0, st>>>(norm, B, totals);
    k_importance<<<(total + 255) / 256, 256, 0, st>>>(norm, totals, B, total, imp_out_dev);
    return fail_cuda("cafe_grad_importance_static");
}

int cafe_migrate(void* h, const void* ids_dev, int ids_are_int64, const int32_t* mask_dev, const int32_t* post_row_dev,
                 int nfields, int B, const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                 float* weight_high, int hotn, int D, int32_t* n_migrated_dev, void* stream) {
    if (!h) return CAFE_ERR_ARG;
    CafeFields F;
    int rc = fill_fields(&F, nfields, B, D, hotn, f_offset, hash_size, weight_hash, weight_high);
    if (rc != CAFE_OK) return rc;
    const int total = nfields * B;
    if (total == 0) return CAFE_OK;
    if (!ids_dev || !mask_dev || !post_row_dev) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t* winner = cafe_internal_ws(h)->row_winner;
    const int blocks = ((total + 31) / 32 + 7) / 8;
    CAFE_PROF(CAFE_P_MIGRATE, st);
    k_migrate_claim<<<(total + 255) / 256, 256, 0, st>>>(mask_dev, post_row_dev, total, winner);
    if (ids_are_int64) k_migrate<int64_t><<<blocks, 256, 0, st>>>(F, (const int64_t*)ids_dev, mask_dev, post_row_dev, total, winner, n_migrated_dev);
    else k_migrate<int32_t><<<blocks, 256, 0, st>>>(F, (const int32_t*)ids_dev, mask_dev, post_row_dev, total, winner, n_migrated_dev);
    return fail_cuda("cafe_migrate");
}

// The scatter in two parts.  scatter_prepare needs only the forward's row numbers (unified row keys and
// their radix sort); scatter_apply reads the sorted keys, the gradient and the tables.  The split lets a
// caller run the first part on the workspace's side stream while the sketch insert runs on the main one.
static int scatter_prepare(CafeEmbedWorkspace* ws, const CafeFields& F, const int32_t* row_dev, int total, int hotn,
                           cudaStream_t st) {
    { CAFE_PROF(CAFE_P_ROWKEYS, st); k_row_keys<<<(total + 255) / 256, 256, 0, st>>>(F, row_dev, total, ws->key[0]); }
    int bits = 1;
    while ((1ll << bits) < (int64_t)hotn + F.hash_base[F.nfields]) ++bits;
    cudaError_t e;
    { CAFE_PROF(CAFE_P_ROWSORT, st);
      // (row key, position) pairs, stable: a row's lookups stay in batch order, which fixes the order of the additions
      CafeKeySource src;
      src.key = ws->key[0]; src.gid = nullptr; src.nb = 0;
      e = cafe_radix_sort(src, nullptr, ws->key_tmp, ws->pos[0], ws->key[1], ws->pos[1], total, bits, ws->sort_scratch, nullptr,
                          nullptr, st); }
    if (e != cudaSuccess) { cafe_internal_set_error(cudaGetErrorString(e)); return CAFE_ERR_CUDA; }
    return CAFE_OK;
}

static int scatter_apply(CafeEmbedWorkspace* ws, const CafeFields& F, const float* grad_dev, int64_t field_stride,
                         int64_t sample_stride, int total, int D, float lr, cudaStream_t st) {
    const int64_t chunks = ((int64_t)total + CAFE_CHUNK - 1) / CAFE_CHUNK;
    { CAFE_PROF(CAFE_P_SCATTER, st);
    DISPATCH_G(D, (k_scatter_chunks<G><<<(unsigned)((chunks * G + 255) / 256), 256, 0, st>>>(F, grad_dev, field_stride,
                   sample_stride, ws->key[1], ws->pos[1], total, lr, ws->partial))); }
    { CAFE_PROF(CAFE_P_FIXUP, st);
    DISPATCH_G(D, (k_scatter_fixup<G><<<(unsigned)((chunks * G + 255) / 256), 256, 0, st>>>(F, ws->key[1], ws->pos[1], total,
                   lr, ws->partial))); }
    return fail_cuda("cafe_scatter_sgd");
}

static int scatter_check(void* h, CafeFields* F, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                         const int32_t* row_dev, int nfields, int B, const int32_t* hash_size, float* const* weight_hash,
                         float* weight_high, int hotn, int D) {
    if (!h) return CAFE_ERR_ARG;
    int64_t zero_off[CAFE_MAX_SEGMENTS] = {0};
    int rc = fill_fields(F, nfields, B, D, hotn, zero_off, hash_size, weight_hash, weight_high);
    if (rc != CAFE_OK) return rc;
    if ((int64_t)nfields * B > cafe_internal_ws(h)->cap) return CAFE_ERR_CAPACITY;
    if (nfields * B > 0 && (!grad_dev || !row_dev || !strides_ok(grad_dev, field_stride, sample_stride))) return CAFE_ERR_ARG;
    return CAFE_OK;
}

int cafe_scatter_sgd(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride,
                     const int32_t* row_dev, int nfields, int B, const int32_t* hash_size, float* const* weight_hash,
                     float* weight_high, int hotn, int D, float lr, void* stream) {
    CafeFields F;
    int rc = scatter_check(h, &F, grad_dev, field_stride, sample_stride, row_dev, nfields, B, hash_size, weight_hash,
                           weight_high, hotn, D);
    if (rc != CAFE_OK) return rc;
    const int total = nfields * B;
    if (total == 0) return CAFE_OK;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    cudaStream_t st = (cudaStream_t)stream;
    rc = scatter_prepare(ws, F, row_dev, total, hotn, st);
    if (rc != CAFE_OK) return rc;
    return scatter_apply(ws, F, grad_dev, field_stride, sample_stride, total, D, lr, st);
}

// Starts scatter_prepare on the side stream, ordered after everything already queued on `st`.
static int scatter_prepare_aside(CafeEmbedWorkspace* ws, const CafeFields& F, const int32_t* row_dev, int total, int hotn,
                                 cudaStream_t st) {
    if (cafe_prof_serialise()) {
        int rc0 = scatter_prepare(ws, F, row_dev, total, hotn, st);
        cudaEventRecord(ws->ev_join, st);
        return rc0;
    }
    if (cudaEventRecord(ws->ev_fork, st) != cudaSuccess || cudaStreamWaitEvent(ws->side, ws->ev_fork, 0) != cudaSuccess)
        return fail_cuda("scatter fork");
    int rc = scatter_prepare(ws, F, row_dev, total, hotn, ws->side);
    // the join is recorded even after a failure so that the main stream never waits on a stale event
    if (cudaEventRecord(ws->ev_join, ws->side) != cudaSuccess) return fail_cuda("scatter join");
    return rc;
}
// Starts (or recognises as already started by cafe_embed_backward_begin) the side work of one backward
// call: the scatter's row sort and, for the parallel insert, the sketch's bucket sorts.
static int backward_side_work(void* h, CafeEmbedWorkspace* ws, const CafeFields& FS, const uint32_t* gid_dev,
                              const int32_t* row_dev, int total, int hotn, int insert_mode, cudaStream_t st) {
    const bool begun = ws->begun_gid == gid_dev && ws->begun_row == row_dev && ws->begun_total == total &&
                       ws->begun_mode == insert_mode && gid_dev != nullptr;
    ws->begun_gid = nullptr; ws->begun_row = nullptr; ws->begun_total = 0;
    if (begun) return CAFE_OK;
    // the sketch's two sorts are queued first (the insert needs them long before the scatter needs the row sort) ...
    if (insert_mode != CAFE_INSERT_SEQUENTIAL) {
        // bucket numbers left by cafe_embed_resolve for exactly these lookups save the sorts their hashing
        const bool have = ws->keys_of == gid_dev && ws->keys_total == total;
        cafe_internal_presort(h, gid_dev, total, have ? ws->bucket_key[0] : nullptr, have ? ws->bucket_key[1] : nullptr, st);
    }
    // ... and run on streams of the highest priority; the row sort's stream has the default one
    const int rc = scatter_prepare_aside(ws, FS, row_dev, total, hotn, st);
    if (rc != CAFE_OK && insert_mode != CAFE_INSERT_SEQUENTIAL) cafe_internal_presort(h, nullptr, 0, nullptr, nullptr, st);   // withdrawn
    return rc;
}
static int scatter_join(CafeEmbedWorkspace* ws, cudaStream_t st) {
    return cudaStreamWaitEvent(st, ws->ev_join, 0) == cudaSuccess ? CAFE_OK : fail_cuda("scatter join wait");
}

// The whole post-backward part of one training step for `nfields` fields, in the reference's order:
// importance -> sketch insert (one call per field, ascending) -> migration with pre-update rows ->
// SGD with the forward-time rows.
// importance of the fields [f0, f0 + nf) of a call over `nfields` fields: the same three kernels as
// cafe_grad_importance, on that range of the workspace
static int importance_range(CafeEmbedWorkspace* ws, const float* grad_dev, int64_t field_stride, int64_t sample_stride, int f0,
                            int nf, int B, int D, float* imp_dev, cudaStream_t st) {
    if (nf <= 0 || B <= 0) return CAFE_OK;
    const int total = nf * B;
    const float* g = grad_dev + (int64_t)f0 * field_stride;
    float* norm = ws->norm + (size_t)f0 * B;
    { CAFE_PROF(CAFE_P_NORM, st);
    DISPATCH_G(D, (k_grad_norm<G><<<(unsigned)((((int64_t)total + 3) / 4 * G + 255) / 256), 256, 0, st>>>(g, field_stride,
                   sample_stride, B, total, norm))); }
    { CAFE_PROF(CAFE_P_FIELDSUM, st); k_field_sum<<<nf, 1024, 0, st>>>(norm, B, ws->totals + f0); }
    { CAFE_PROF(CAFE_P_IMPORTANCE, st); k_importance<<<(total + 255) / 256, 256, 0, st>>>(norm, ws->totals + f0, B, total,
                                                                                           imp_dev + (size_t)f0 * B); }
    return fail_cuda("cafe_grad_importance");
}

// gate_field in (0, nfields) with a gate event: the gradient rows of the fields from gate_field on are
// being written by work that `stream` has not waited for; they are complete once gate_event has fired.
static int embed_backward_impl(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride, const void* ids_dev,
                               int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev, int nfields, int B,
                               const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                               float* weight_high, int hotn, int D, float lr, int insert_mode, int32_t* mask_out_dev,
                               int32_t* n_migrated_dev, int gate_field, cudaEvent_t gate_event, cudaStream_t st) {
    if (!h) return CAFE_ERR_ARG;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    const int64_t total = (int64_t)nfields * B;
    if (total > ws->cap) return CAFE_ERR_CAPACITY;
    if (total == 0) return CAFE_OK;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    CafeFields FS;
    int rc = scatter_check(h, &FS, grad_dev, field_stride, sample_stride, row_dev, nfields, B, hash_size, weight_hash,
                           weight_high, hotn, D);
    if (rc != CAFE_OK) return rc;
    bool gated = gate_event != nullptr && gate_field > 0 && gate_field < nfields;
    if (gate_event != nullptr && (!gated || cafe_prof_serialise())) {
        // nothing to overlap (or per-kernel timing is on): simply wait for the late fields first
        if (cudaStreamWaitEvent(st, gate_event, 0) != cudaSuccess) return fail_cuda("gate wait");
        gated = false;
    }
    rc = backward_side_work(h, ws, FS, gid_dev, row_dev, (int)total, hotn, insert_mode, st);
    if (rc != CAFE_OK) { scatter_join(ws, st); return rc; }
    const int early = gated ? gate_field : nfields;
    rc = importance_range(ws, grad_dev, field_stride, sample_stride, 0, early, B, D, ws->imp, st);
    if (rc == CAFE_OK && gated) {
        // the late fields' importance runs on a stream of its own, behind the gate; the insert waits for it
        // only when it reaches those fields
        if (cudaStreamWaitEvent(ws->late, gate_event, 0) != cudaSuccess) rc = fail_cuda("gate wait");
        if (rc == CAFE_OK) rc = importance_range(ws, grad_dev, field_stride, sample_stride, gate_field, nfields - gate_field, B, D,
                                                 ws->imp, ws->late);
        if (cudaEventRecord(ws->ev_late, ws->late) != cudaSuccess && rc == CAFE_OK) rc = fail_cuda("gate record");
        if (rc == CAFE_OK) cafe_internal_set_gate(h, gate_field, ws->ev_late);
    }
    if (rc != CAFE_OK) {
        cafe_internal_presort(h, nullptr, 0, nullptr, nullptr, st);   // withdraws the sorts started above
        scatter_join(ws, st);
        return rc;
    }
    int seg[CAFE_MAX_SEGMENTS + 1];
    for (int f = 0; f <= nfields; ++f) seg[f] = f * B;
    int32_t* mask = mask_out_dev ? mask_out_dev : ws->mask;
    int status = cafe_internal_insert(h, gid_dev, ws->imp, seg, nfields, mask, ws->post_row, insert_mode, st);
    cafe_internal_set_gate(h, -1, nullptr);
    if (gated) cudaStreamWaitEvent(st, ws->ev_late, 0);   // whatever the insert did: the scatter reads every field
    rc = scatter_join(ws, st);
    if (status != CAFE_OK && status != CAFE_ERR_NOCONVERGE && status != CAFE_ERR_RESET_UNDERFLOW) return status;
    if (rc != CAFE_OK) return rc;
    rc = cafe_migrate(h, ids_dev, ids_are_int64, mask, ws->post_row, nfields, B, f_offset, hash_size, weight_hash, weight_high,
                      hotn, D, n_migrated_dev, st);
    if (rc != CAFE_OK) return rc;
    rc = scatter_apply(ws, FS, grad_dev, field_stride, sample_stride, (int)total, D, lr, st);
    return rc != CAFE_OK ? rc : status;
}

int cafe_embed_backward(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride, const void* ids_dev,
                        int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev, int nfields, int B,
                        const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash, float* weight_high,
                        int hotn, int D, float lr, int insert_mode, int32_t* mask_out_dev, int32_t* n_migrated_dev,
                        void* stream) {
    return embed_backward_impl(h, grad_dev, field_stride, sample_stride, ids_dev, ids_are_int64, gid_dev, row_dev, nfields, B,
                               f_offset, hash_size, weight_hash, weight_high, hotn, D, lr, insert_mode, mask_out_dev,
                               n_migrated_dev, 0, nullptr, (cudaStream_t)stream);
}

int cafe_embed_backward_gated(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride, const void* ids_dev,
                              int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev, int nfields, int B,
                              const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                              float* weight_high, int hotn, int D, float lr, int insert_mode, int gate_field,
                              void* gate_event, void* stream) {
    if (!gate_event) return CAFE_ERR_ARG;
    return embed_backward_impl(h, grad_dev, field_stride, sample_stride, ids_dev, ids_are_int64, gid_dev, row_dev, nfields, B,
                               f_offset, hash_size, weight_hash, weight_high, hotn, D, lr, insert_mode, nullptr, nullptr,
                               gate_field, (cudaEvent_t)gate_event, (cudaStream_t)stream);
}

// ---- field-sharded exchange over peer memory (see the kernels above) ------------------------------
int cafe_shard_scatter_ids(const int64_t* ids_local_dev, int nfields_total, int rows_local, int nranks, int rank,
                           int64_t* const* owner_ids, void* stream) {
    if (nfields_total < 1 || rows_local < 0 || nranks < 1 || nranks > CAFE_MAX_RANKS || rank < 0 || rank >= nranks || !owner_ids)
        return CAFE_ERR_ARG;
    const int64_t total = (int64_t)nfields_total * rows_local;
    if (total == 0) return CAFE_OK;
    if (!ids_local_dev) return CAFE_ERR_ARG;
    CafeIdBuffers d;
    memset(&d, 0, sizeof(d));
    for (int r = 0; r < nranks; ++r) { if (!owner_ids[r]) return CAFE_ERR_ARG; d.base[r] = owner_ids[r]; }
    cudaStream_t st = (cudaStream_t)stream;
    CAFE_PROF(CAFE_P_IDS, st);
    k_scatter_ids<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(ids_local_dev, nfields_total, rows_local, nranks, rank, d);
    return fail_cuda("cafe_shard_scatter_ids");
}

int cafe_embed_forward_sharded(void* h, const void* ids_dev, int ids_are_int64, int nfields, int B, const int64_t* f_offset,
                               const int32_t* hash_size, float* const* weight_hash, float* weight_high, int hotn, int D,
                               float* const* out_rank, int nranks, int rows_per_rank, int64_t out_field_stride,
                               int64_t out_sample_stride, uint32_t* gid_out_dev, int32_t* row_out_dev, void* stream) {
    if (!h || !out_rank || nranks < 1 || nranks > CAFE_MAX_RANKS || rows_per_rank < 1) return CAFE_ERR_ARG;
    if ((int64_t)rows_per_rank * nranks != B) return CAFE_ERR_ARG;
    CafeFields F;
    int rc = fill_fields(&F, nfields, B, D, hotn, f_offset, hash_size, weight_hash, weight_high);
    if (rc != CAFE_OK) return rc;
    const int total = nfields * B;
    if (total == 0) return CAFE_OK;
    if (!ids_dev || !gid_out_dev || !row_out_dev || out_field_stride % 4 || out_sample_stride % 4) return CAFE_ERR_ARG;
    CafeRankBuffers ob;
    memset(&ob, 0, sizeof(ob));
    for (int r = 0; r < nranks; ++r) { if (!out_rank[r] || !aligned16(out_rank[r])) return CAFE_ERR_ARG; ob.base[r] = out_rank[r]; }
    ob.rows_per_rank = rows_per_rank;
    CafeSketchView V = cafe_internal_view(h);
    if (hotn != V.lim) return CAFE_ERR_ARG;
    return launch_forward(F, ids_dev, ids_are_int64, V, ob, out_field_stride, out_sample_stride, gid_out_dev, row_out_dev, total, D,
                          (cudaStream_t)stream);
}

int cafe_shard_pull_importance(void* h, const float* const* grad_rank, int nranks, int rows_per_rank, int nfields, int D,
                               int64_t field_stride, int64_t sample_stride, float* local_grad_dev, float* imp_out_dev,
                               void* stream) {
    if (!h || !grad_rank || nranks < 1 || nranks > CAFE_MAX_RANKS || rows_per_rank < 1 || nfields < 1 || nfields > CAFE_MAX_SEGMENTS)
        return CAFE_ERR_ARG;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    const int B = rows_per_rank * nranks;
    const int64_t total64 = (int64_t)nfields * B;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    if (total64 > ws->cap) return CAFE_ERR_CAPACITY;
    if (!local_grad_dev || !imp_out_dev || !strides_ok(local_grad_dev, field_stride, sample_stride)) return CAFE_ERR_ARG;
    CafeRankBuffers sb;
    memset(&sb, 0, sizeof(sb));
    for (int r = 0; r < nranks; ++r) { if (!grad_rank[r] || !aligned16(grad_rank[r])) return CAFE_ERR_ARG; sb.base[r] = const_cast<float*>(grad_rank[r]); }
    sb.rows_per_rank = rows_per_rank;
    const int total = (int)total64;
    cudaStream_t st = (cudaStream_t)stream;
    { CAFE_PROF(CAFE_P_NORM, st);
    DISPATCH_G(D, (k_pull_norm<G><<<(unsigned)((((int64_t)total + 3) / 4 * G + 255) / 256), 256, 0, st>>>(sb, field_stride,
                   sample_stride, B, total, local_grad_dev, ws->norm))); }
    { CAFE_PROF(CAFE_P_FIELDSUM, st); k_field_sum<<<nfields, 1024, 0, st>>>(ws->norm, B, ws->totals); }
    { CAFE_PROF(CAFE_P_IMPORTANCE, st); k_importance<<<(total + 255) / 256, 256, 0, st>>>(ws->norm, ws->totals, B, total, imp_out_dev); }
    return fail_cuda("cafe_shard_pull_importance");
}

int cafe_embed_backward_begin(void* h, const uint32_t* gid_dev, const int32_t* row_dev, int nfields, int B,
                              const int32_t* hash_size, float* const* weight_hash, float* weight_high, int hotn, int D,
                              int insert_mode, void* stream) {
    if (!h || !gid_dev || !row_dev) return CAFE_ERR_ARG;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    CafeFields FS;
    int64_t zero_off[CAFE_MAX_SEGMENTS] = {0};
    int rc = fill_fields(&FS, nfields, B, D, hotn, zero_off, hash_size, weight_hash, weight_high);
    if (rc != CAFE_OK) return rc;
    const int64_t total = (int64_t)nfields * B;
    if (total > ws->cap) return CAFE_ERR_CAPACITY;
    if (total == 0) return CAFE_OK;
    ws->begun_gid = nullptr;
    rc = backward_side_work(h, ws, FS, gid_dev, row_dev, (int)total, hotn, insert_mode, (cudaStream_t)stream);
    if (rc != CAFE_OK) return rc;
    ws->begun_gid = gid_dev; ws->begun_row = row_dev; ws->begun_total = (int)total; ws->begun_mode = insert_mode;
    return CAFE_OK;
}

// cafe_embed_backward with the importance array already computed (by cafe_shard_pull_importance)
int cafe_embed_backward_imp(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride, const float* imp_dev,
                            const void* ids_dev, int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev,
                            int nfields, int B, const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                            float* weight_high, int hotn, int D, float lr, int insert_mode, int32_t* mask_out_dev,
                            void* stream) {
    if (!h || !imp_dev) return CAFE_ERR_ARG;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    const int64_t total = (int64_t)nfields * B;
    if (nfields < 1 || nfields > CAFE_MAX_SEGMENTS || total > ws->cap) return CAFE_ERR_CAPACITY;
    if (total == 0) return CAFE_OK;
    int seg[CAFE_MAX_SEGMENTS + 1];
    for (int f = 0; f <= nfields; ++f) seg[f] = f * B;
    int32_t* mask = mask_out_dev ? mask_out_dev : ws->mask;
    CafeFields FS;
    int rc = scatter_check(h, &FS, grad_dev, field_stride, sample_stride, row_dev, nfields, B, hash_size, weight_hash,
                           weight_high, hotn, D);
    if (rc != CAFE_OK) return rc;
    rc = backward_side_work(h, ws, FS, gid_dev, row_dev, (int)total, hotn, insert_mode, (cudaStream_t)stream);
    if (rc != CAFE_OK) { scatter_join(ws, (cudaStream_t)stream); return rc; }
    int status = cafe_internal_insert(h, gid_dev, imp_dev, seg, nfields, mask, ws->post_row, insert_mode, (cudaStream_t)stream);
    rc = scatter_join(ws, (cudaStream_t)stream);
    if (status != CAFE_OK && status != CAFE_ERR_NOCONVERGE && status != CAFE_ERR_RESET_UNDERFLOW) return status;
    if (rc != CAFE_OK) return rc;
    rc = cafe_migrate(h, ids_dev, ids_are_int64, mask, ws->post_row, nfields, B, f_offset, hash_size, weight_hash, weight_high,
                      hotn, D, nullptr, stream);
    if (rc != CAFE_OK) return rc;
    rc = scatter_apply(ws, FS, grad_dev, field_stride, sample_stride, (int)total, D, lr, (cudaStream_t)stream);
    return rc != CAFE_OK ? rc : status;
}

static int push_grads_impl(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks, int rank,
                           float* const* owner_grad, int j_begin, int j_end, void* stream) {
    if (nfields_total < 1 || rows_local < 0 || nranks < 1 || nranks > CAFE_MAX_RANKS || rank < 0 || rank >= nranks || !owner_grad)
        return CAFE_ERR_ARG;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    const int64_t total_rows = (int64_t)nfields_total * rows_local;
    if (total_rows == 0) return CAFE_OK;
    if (!grad_blocked_dev || !aligned16(grad_blocked_dev)) return CAFE_ERR_ARG;
    CafePushPlan P;
    memset(&P, 0, sizeof(P));
    int64_t off = 0;
    for (int g = 0; g < nranks; ++g) {
        if (!owner_grad[g] || !aligned16(owner_grad[g])) return CAFE_ERR_ARG;
        P.base[g] = owner_grad[g];
        P.fields_of[g] = nfields_total / nranks + (g < nfields_total % nranks ? 1 : 0);   // round-robin ownership
        P.row_off[g] = (int32_t)off;
        off += (int64_t)P.fields_of[g] * rows_local;
    }
    P.row_off[nranks] = (int32_t)off;
    if (off != total_rows || total_rows > 0x7fffffffLL) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    CAFE_PROF(CAFE_P_PUSH, st);
    const int64_t threads = total_rows * (D / 4);
    const int64_t blocks = (threads + 255) / 256;
    k_push_grads<<<(unsigned)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(grad_blocked_dev, P, nranks, rank, rows_local, D,
                                                                                 total_rows, j_begin, j_end);
    return fail_cuda("cafe_shard_push_grads");
}

int cafe_shard_push_norms(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks, int rank,
                          float* const* owner_norm, float* staging_dev, void* stream) {
    if (nfields_total < 1 || rows_local < 0 || nranks < 1 || nranks > CAFE_MAX_RANKS || rank < 0 || rank >= nranks || !owner_norm ||
        !staging_dev)
        return CAFE_ERR_ARG;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return CAFE_ERR_UNSUPPORTED;
    const int64_t total_rows = (int64_t)nfields_total * rows_local;
    if (total_rows == 0) return CAFE_OK;
    if (!grad_blocked_dev || !aligned16(grad_blocked_dev)) return CAFE_ERR_ARG;
    CafePushPlan P;
    memset(&P, 0, sizeof(P));
    int64_t off = 0;
    for (int g = 0; g < nranks; ++g) {
        if (!owner_norm[g]) return CAFE_ERR_ARG;
        P.base[g] = owner_norm[g];
        P.fields_of[g] = nfields_total / nranks + (g < nfields_total % nranks ? 1 : 0);   // round-robin ownership
        P.row_off[g] = (int32_t)off;
        off += (int64_t)P.fields_of[g] * rows_local;
    }
    P.row_off[nranks] = (int32_t)off;
    if (off != total_rows || total_rows > 0x7fffffffLL) return CAFE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    CAFE_PROF(CAFE_P_NORM, st);
    DISPATCH_G(D, (k_push_norms<G><<<(unsigned)(((total_rows + 3) / 4 * G + 255) / 256), 256, 0, st>>>(grad_blocked_dev, P, nranks,
                   rows_local, total_rows, staging_dev)));
    k_send_norms<<<(unsigned)((total_rows + 255) / 256), 256, 0, st>>>(staging_dev, P, nranks, rank, rows_local, total_rows);
    return fail_cuda("cafe_shard_push_norms");
}

// cafe_embed_backward with the lookups' gradient norms already at hand (cafe_shard_push_norms) and the gradient rows
// possibly still on their way: importance and the sketch insert run at once from the norms; the stream waits for
// gate_event (null = the rows are there) only before the step that reads the rows, the SGD scatter.
int cafe_embed_backward_norms(void* h, const float* grad_dev, int64_t field_stride, int64_t sample_stride, const float* norm_dev,
                              const void* ids_dev, int ids_are_int64, const uint32_t* gid_dev, const int32_t* row_dev,
                              int nfields, int B, const int64_t* f_offset, const int32_t* hash_size, float* const* weight_hash,
                              float* weight_high, int hotn, int D, float lr, int insert_mode, void* gate_event, void* stream) {
    if (!h || !norm_dev) return CAFE_ERR_ARG;
    CafeEmbedWorkspace* ws = cafe_internal_ws(h);
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t total = (int64_t)nfields * B;
    if (nfields < 1 || nfields > CAFE_MAX_SEGMENTS || total > ws->cap) return CAFE_ERR_CAPACITY;
    if (total == 0) return CAFE_OK;
    CafeFields FS;
    int rc = scatter_check(h, &FS, grad_dev, field_stride, sample_stride, row_dev, nfields, B, hash_size, weight_hash,
                           weight_high, hotn, D);
    if (rc != CAFE_OK) return rc;
    rc = backward_side_work(h, ws, FS, gid_dev, row_dev, (int)total, hotn, insert_mode, st);
    if (rc != CAFE_OK) { scatter_join(ws, st); return rc; }
    { CAFE_PROF(CAFE_P_FIELDSUM, st); k_field_sum<<<nfields, 1024, 0, st>>>(norm_dev, B, ws->totals); }
    { CAFE_PROF(CAFE_P_IMPORTANCE, st); k_importance<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(norm_dev, ws->totals, B,
                                                                                                    (int)total, ws->imp); }
    int seg[CAFE_MAX_SEGMENTS + 1];
    for (int f = 0; f <= nfields; ++f) seg[f] = f * B;
    int status = cafe_internal_insert(h, gid_dev, ws->imp, seg, nfields, ws->mask, ws->post_row, insert_mode, st);
    rc = scatter_join(ws, st);
    if (status != CAFE_OK && status != CAFE_ERR_NOCONVERGE && status != CAFE_ERR_RESET_UNDERFLOW) return status;
    if (rc != CAFE_OK) return rc;
    rc = cafe_migrate(h, ids_dev, ids_are_int64, ws->mask, ws->post_row, nfields, B, f_offset, hash_size, weight_hash, weight_high,
                      hotn, D, nullptr, stream);
    if (rc != CAFE_OK) return rc;
    if (gate_event && cudaStreamWaitEvent(st, (cudaEvent_t)gate_event, 0) != cudaSuccess) return fail_cuda("gate wait");
    rc = scatter_apply(ws, FS, grad_dev, field_stride, sample_stride, (int)total, D, lr, st);
    return rc != CAFE_OK ? rc : status;
}

int cafe_shard_push_grads(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks, int rank,
                          float* const* owner_grad, void* stream) {
    return push_grads_impl(grad_blocked_dev, nfields_total, rows_local, D, nranks, rank, owner_grad, 0, 0x7fffffff, stream);
}

int cafe_shard_push_grads_fields(const float* grad_blocked_dev, int nfields_total, int rows_local, int D, int nranks, int rank,
                                 float* const* owner_grad, int j_begin, int j_end, void* stream) {
    if (j_begin < 0 || j_end < j_begin) return CAFE_ERR_ARG;
    return push_grads_impl(grad_blocked_dev, nfields_total, rows_local, D, nranks, rank, owner_grad, j_begin, j_end, stream);
}

}  // extern "C"
