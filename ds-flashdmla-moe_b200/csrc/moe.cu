// MoE FFN plumbing around the expert GEMMs: top-k gate, per-expert packing (bucket + exclusive scan),
// row gather and weighted combine.  These are the pieces the reference lists as csrc/moe/router_topk.cu,
// pack_dispatch.cu and combine_scatter.cu (README.md:17-20, 48-53; none of them is shipped).  All four are
// HBM-bound integer / row-copy work on CUDA cores; the packing is deterministic (assignments keep their
// token order inside an expert), so its outputs are compared bit for bit.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/flashdmla.h"

namespace fdmla {
namespace moe {

constexpr int PACK_BLOCK = 256;       // assignments per block of the packing pass

// ---- gate: one warp per token --------------------------------------------------------------------
// p = softmax(logits) over E experts; the k largest win (ties: lower index), listed by descending p;
// w = p / sum of the selected p.
__global__ void route_topk_kernel(const float *__restrict__ logits, int *__restrict__ idx, float *__restrict__ w,
                                  int T, int E, int k) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const float *row = logits + (size_t)t * E;
    float mx = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, row[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += __expf(row[e] - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    // k rounds of arg-max over the logits (same order as over p); winners are excluded by index
    float sel_sum = 0.f;
    float my_w = 0.f;                 // lane j keeps the j-th winner
    int my_i = -1;
    unsigned long long taken_lo = 0;  // this lane's own experts already taken (bit per stride step, E <= 2048)
    for (int j = 0; j < k; ++j) {
        float bv = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int e = lane, s = 0; e < E; e += 32, ++s) {
            if ((taken_lo >> s) & 1ull) continue;
            const float v = row[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((bi & 31) == lane) taken_lo |= 1ull << (bi >> 5);
        const float pj = __expf(bv - mx) / sum;
        sel_sum += pj;
        if (lane == j) { my_w = pj; my_i = bi; }
    }
    if (lane < k) {
        idx[(size_t)t * k + lane] = my_i;
        w[(size_t)t * k + lane] = my_w / sel_sum;
    }
}

// ---- packing, pass 1: per-block expert counts and each assignment's rank inside its block ----------
__global__ void __launch_bounds__(PACK_BLOCK) pack_count_kernel(const int *__restrict__ idx, int *__restrict__ blk_counts,
                                                                int *__restrict__ local_rank, int A, int E) {
    __shared__ int s_e[PACK_BLOCK];
    extern __shared__ int s_hist[];
    const int a = blockIdx.x * PACK_BLOCK + threadIdx.x;
    int e = -1;
    if (a < A) {
        e = idx[a];
        if (e < 0 || e >= E) e = -1;          // a bad expert id is dropped, never written through
    }
    s_e[threadIdx.x] = e;
    for (int i = threadIdx.x; i < E; i += PACK_BLOCK) s_hist[i] = 0;
    __syncthreads();
    if (e >= 0) {
        int r = 0;
        for (int i = 0; i < (int)threadIdx.x; ++i) r += (s_e[i] == e);
        local_rank[a] = r;
        atomicAdd(&s_hist[e], 1);
    } else if (a < A) {
        local_rank[a] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < E; i += PACK_BLOCK) blk_counts[(size_t)blockIdx.x * E + i] = s_hist[i];
}

// ---- pass 2a: one warp per expert turns the per-block counts into each block's first rank inside the expert -
__global__ void pack_scan_blocks_kernel(int *__restrict__ blk_counts, int *__restrict__ totals, int n_blocks, int E, int capacity) {
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (e >= E) return;
    int run = 0;
    for (int b0 = 0; b0 < n_blocks; b0 += 32) {
        const int b = b0 + lane;
        const int c = b < n_blocks ? blk_counts[(size_t)b * E + e] : 0;
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (b < n_blocks) blk_counts[(size_t)b * E + e] = run + incl - c;
        run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[e] = run < capacity ? run : capacity;
}

// ---- pass 2b (one block): exclusive scan of the kept counts over the experts -------------------------------
// (padded: every expert owns `capacity` rows, offsets[e] = e * capacity, so that the packed rows are an [E, capacity, d] batch)
__global__ void pack_scan_experts_kernel(const int *__restrict__ totals, int *__restrict__ offsets, int E, int capacity, int padded) {
    __shared__ int s_part[256];
    if (padded) {
        for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = e * capacity;
        return;
    }
    const int per = (E + 255) / 256, lo = threadIdx.x * per, hi = lo + per < E ? lo + per : E;
    int sum = 0;
    for (int e = lo; e < hi; ++e) sum += totals[e];
    s_part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < 256; ++i) { const int c = s_part[i]; s_part[i] = run; run += c; }
        offsets[E] = run;
    }
    __syncthreads();
    int run = s_part[threadIdx.x];
    for (int e = lo; e < hi; ++e) { offsets[e] = run; run += totals[e]; }
}

// ---- pass 3: packed position of every assignment and the token of every packed row ------------------
__global__ void __launch_bounds__(PACK_BLOCK) pack_assign_kernel(const int *__restrict__ idx, const int *__restrict__ blk_first,
                                                                 const int *__restrict__ local_rank, const int *__restrict__ offsets,
                                                                 int *__restrict__ pos, int *__restrict__ perm, int A, int E, int k,
                                                                 int capacity) {
    const int a = blockIdx.x * PACK_BLOCK + threadIdx.x;
    if (a >= A) return;
    const int lr = local_rank[a];
    int p = -1;
    if (lr >= 0) {
        const int e = idx[a];
        const int r = blk_first[(size_t)blockIdx.x * E + e] + lr;
        if (r < capacity) {
            p = offsets[e] + r;
            perm[p] = a / k;
        }
    }
    pos[a] = p;
}

// The gather walks its 16-byte vectors flat over a grid that fills the GPU once, keeps (row, vector) as a pair that
// advances by the grid's stride - no division in the loop - and issues several loads before the first store.
struct RowVec {
    int r, v;                    // row and vector inside the row
    int dr, dv, vpr;             // the grid's stride as (rows, vectors), vectors per row
    __device__ __forceinline__ RowVec(int vec_per_row) : vpr(vec_per_row) {
        const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x, st = (long long)gridDim.x * blockDim.x;
        r = (int)(i / vpr); v = (int)(i - (long long)r * vpr);
        dr = (int)(st / vpr); dv = (int)(st - (long long)dr * vpr);
    }
    __device__ __forceinline__ void step() {
        r += dr; v += dv;
        if (v >= vpr) { v -= vpr; ++r; }
    }
};

// ---- gather: packed[r] = x[perm[r]] (16-byte vectors) -----------------------------------------------
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4 *__restrict__ x, const int *__restrict__ perm,
                                                          const int *__restrict__ offsets, uint4 *__restrict__ packed, int E,
                                                          int vec_per_row) {
    const int n_rows = offsets[E];
    constexpr int U = 4;
    RowVec it(vec_per_row);
    while (it.r < n_rows) {
        uint4 val[U];
        size_t dst[U];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            live[u] = it.r < n_rows;
            val[u] = make_uint4(0, 0, 0, 0);
            if (live[u]) {
                dst[u] = (size_t)it.r * vec_per_row + it.v;
                const int t = perm[it.r];          // -1: a row of padded packing that holds no assignment
                if (t >= 0) val[u] = x[(size_t)t * vec_per_row + it.v];
            }
            it.step();
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (live[u]) packed[dst[u]] = val[u];
    }
}

// ---- scatter: packed[pos[t,j]] = x[t] for every kept assignment: each token row is read once and written to
// its (up to k) packed rows, so HBM sees T + rows rows instead of the 2 x rows of the gather above when the
// packed rows stream the token rows out of L2 ---------------------------------------------------------------
__global__ void scatter_rows_kernel(const uint4 *__restrict__ x, const int *__restrict__ pos, uint4 *__restrict__ packed, int T,
                                    int k, int vec_per_row) {
    __shared__ int s_pos[32];
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < k) s_pos[threadIdx.x] = pos[(size_t)t * k + threadIdx.x];
        __syncthreads();
        constexpr int U = 4;            // vectors of the row a thread reads before it starts storing
        for (int v0 = threadIdx.x; v0 < vec_per_row; v0 += blockDim.x * U) {
            uint4 val[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int v = v0 + u * blockDim.x;
                if (v < vec_per_row) val[u] = x[(size_t)t * vec_per_row + v];
            }
            for (int j = 0; j < k; ++j) {
                const int p = s_pos[j];
                if (p < 0) continue;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int v = v0 + u * blockDim.x;
                    if (v < vec_per_row) packed[(size_t)p * vec_per_row + v] = val[u];
                }
            }
        }
    }
}

// ---- combine: out[t] = sum_j w'[t,j] y[pos[t,j]] (+ shared[t]); w' = kept weights rescaled to sum 1 ---
template <typename TX>
__global__ void combine_kernel(const TX *__restrict__ y, const int *__restrict__ pos, const float *__restrict__ w,
                               const TX *__restrict__ shared, TX *__restrict__ out, int T, int k, int d) {
    const int t = blockIdx.x;
    if (t >= T) return;
    float kept_sum = 0.f;
    for (int j = 0; j < k; ++j) kept_sum += pos[(size_t)t * k + j] >= 0 ? w[(size_t)t * k + j] : 0.f;
    const float inv = kept_sum > 0.f ? 1.f / kept_sum : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < k; ++j) {
            const int p = pos[(size_t)t * k + j];
            if (p >= 0) acc += w[(size_t)t * k + j] * inv * (float)y[(size_t)p * d + c];
        }
        if (shared) acc += (float)shared[(size_t)t * d + c];
        out[(size_t)t * d + c] = (TX)acc;
    }
}

// bf16 rows whose length is a multiple of 8 and whose bases are 16-byte aligned: 16-byte vectors, the k source
// rows of a token read side by side
__global__ void combine_bf16x8_kernel(const __nv_bfloat16 *__restrict__ y, const int *__restrict__ pos, const float *__restrict__ w,
                                      const __nv_bfloat16 *__restrict__ shared, __nv_bfloat16 *__restrict__ out, int T, int k,
                                      int d) {
    __shared__ int s_pos[32];
    __shared__ float s_w[32];
    const int t = blockIdx.x;
    if (threadIdx.x < k) {
        const int p = pos[(size_t)t * k + threadIdx.x];
        s_pos[threadIdx.x] = p;
        s_w[threadIdx.x] = p >= 0 ? w[(size_t)t * k + threadIdx.x] : 0.f;
    }
    __syncthreads();
    float kept_sum = 0.f;
    for (int j = 0; j < k; ++j) kept_sum += s_w[j];
    const float inv = kept_sum > 0.f ? 1.f / kept_sum : 0.f;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        constexpr int U = 8;            // source rows read side by side: all of their loads are issued before the sums
        for (int j0 = 0; j0 < k; j0 += U) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int p = j0 + u < k ? s_pos[j0 + u] : -1;
                if (p >= 0) v[u] = *reinterpret_cast<const uint4 *>(y + (size_t)p * d + c);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (j0 + u >= k || s_pos[j0 + u] < 0) continue;
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v[u]);
                const float wj = s_w[j0 + u] * inv;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(h[e]);
                    acc[2 * e] += wj * f.x;
                    acc[2 * e + 1] += wj * f.y;
                }
            }
        }
        if (shared) {
            const uint4 v = *reinterpret_cast<const uint4 *>(shared + (size_t)t * d + c);
            const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                acc[2 * e] += f.x;
                acc[2 * e + 1] += f.y;
            }
        }
        uint4 o;
        __nv_bfloat162 *ho = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) ho[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        *reinterpret_cast<uint4 *>(out + (size_t)t * d + c) = o;
    }
}

static int launch_ok() { return cudaGetLastError() == cudaSuccess ? FDMLA_OK : FDMLA_ERR_CUDA; }

}  // namespace moe
}  // namespace fdmla

using namespace fdmla::moe;

extern "C" int fdmla_moe_route_topk(const float *logits, int *idx, float *w, int T, int E, int k, void *stream) {
    if (!logits || !idx || !w || T < 0 || E <= 0 || k <= 0) return FDMLA_ERR_INVALID;
    if (k > E || k > 32 || E > 2048) return FDMLA_ERR_UNSUPPORTED;
    if (T == 0) return FDMLA_OK;
    const int warps = 4;
    route_topk_kernel<<<(T + warps - 1) / warps, warps * 32, 0, (cudaStream_t)stream>>>(logits, idx, w, T, E, k);
    return launch_ok();
}

extern "C" size_t fdmla_moe_pack_workspace_bytes(int T, int k, int E) {
    if (T < 0 || k <= 0 || E <= 0) return 0;
    const long long A = (long long)T * k, nb = (A + PACK_BLOCK - 1) / PACK_BLOCK;
    return (size_t)((nb > 0 ? nb : 1) * E + (A > 0 ? A : 1) + E) * sizeof(int);
}

extern "C" int fdmla_moe_pack(const int *idx, int *pos, int *perm, int *offsets, void *workspace, size_t workspace_bytes,
                              int T, int k, int E, int capacity, int padded, void *stream) {
    if (!idx || !pos || !perm || !offsets || T < 0 || k <= 0 || E <= 0 || capacity < 0) return FDMLA_ERR_INVALID;
    if (padded && (long long)E * capacity > 0x7fffffffLL) return FDMLA_ERR_UNSUPPORTED;
    if (E > 8192) return FDMLA_ERR_UNSUPPORTED;                  // the per-block histogram lives in shared memory
    if (!workspace || workspace_bytes < fdmla_moe_pack_workspace_bytes(T, k, E)) return FDMLA_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    const int A = T * k, nb = (A + PACK_BLOCK - 1) / PACK_BLOCK;
    int *blk = static_cast<int *>(workspace), *lrank = blk + (size_t)(nb > 0 ? nb : 1) * E, *totals = lrank + (A > 0 ? A : 1);
    // padded packing: rows past an expert's count keep no token; mark them so that a gather skips them
    if (padded && (size_t)E * capacity > 0 &&
        cudaMemsetAsync(perm, 0xff, (size_t)E * capacity * sizeof(int), s) != cudaSuccess) return FDMLA_ERR_CUDA;
    if (nb > 0) pack_count_kernel<<<nb, PACK_BLOCK, E * sizeof(int), s>>>(idx, blk, lrank, A, E);
    pack_scan_blocks_kernel<<<(E + 7) / 8, 256, 0, s>>>(blk, totals, nb, E, capacity);
    pack_scan_experts_kernel<<<1, 256, 0, s>>>(totals, offsets, E, capacity, padded);
    if (nb > 0) pack_assign_kernel<<<nb, PACK_BLOCK, 0, s>>>(idx, blk, lrank, offsets, pos, perm, A, E, k, capacity);
    return launch_ok();
}

extern "C" int fdmla_moe_gather(const void *x, const int *perm, const int *offsets, void *packed, int max_rows, int E, int d,
                                int dtype, void *stream) {
    if (!x || !perm || !offsets || !packed || max_rows < 0 || E <= 0 || d <= 0) return FDMLA_ERR_INVALID;
    const int esz = dtype == FDMLA_BF16 ? 2 : (dtype == FDMLA_F32 ? 4 : 0);
    if (!esz) return FDMLA_ERR_INVALID;
    if ((d * esz) % 16 || ((uintptr_t)x | (uintptr_t)packed) % 16) return FDMLA_ERR_UNSUPPORTED;
    if (max_rows == 0) return FDMLA_OK;
    const int vec = d * esz / 16;
    // four vectors per thread and round; at most the blocks that are resident at once (one wave, no tail)
    static int resident = 0;
    if (resident == 0) {
        int per_sm = 0, dev = 0, sms = 148;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gather_rows_kernel, 256, 0) != cudaSuccess || per_sm < 1) {
            cudaGetLastError();
            per_sm = 4;
        }
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            cudaGetLastError();
            sms = 148;
        }
        resident = per_sm * sms;
    }
    long long blocks = ((long long)max_rows * vec + 1023) / 1024;
    if (blocks > resident) blocks = resident;
    if (blocks < 1) blocks = 1;
    gather_rows_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4 *>(x), perm, offsets,
                                                                      static_cast<uint4 *>(packed), E, vec);
    return launch_ok();
}

extern "C" int fdmla_moe_scatter(const void *x, const int *pos, void *packed, int T, int k, int d, int dtype, void *stream) {
    if (!x || !pos || !packed || T < 0 || k <= 0 || d <= 0) return FDMLA_ERR_INVALID;
    const int esz = dtype == FDMLA_BF16 ? 2 : (dtype == FDMLA_F32 ? 4 : 0);
    if (!esz) return FDMLA_ERR_INVALID;
    if (k > 32 || (d * esz) % 16 || ((uintptr_t)x | (uintptr_t)packed) % 16) return FDMLA_ERR_UNSUPPORTED;
    if (T == 0) return FDMLA_OK;
    const int vec = d * esz / 16;
    const int blocks = T < 148 * 8 ? T : 148 * 8;
    scatter_rows_kernel<<<blocks, vec >= 256 ? 256 : 128, 0, (cudaStream_t)stream>>>(static_cast<const uint4 *>(x), pos,
                                                                                    static_cast<uint4 *>(packed), T, k, vec);
    return launch_ok();
}

extern "C" int fdmla_moe_combine(const void *y, const int *pos, const float *w, const void *shared, void *out, int T, int k,
                                 int d, int dtype, void *stream) {
    if (!y || !pos || !w || !out || T < 0 || k <= 0 || d <= 0) return FDMLA_ERR_INVALID;
    if (dtype != FDMLA_BF16 && dtype != FDMLA_F32) return FDMLA_ERR_INVALID;
    if (T == 0) return FDMLA_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec_ok = dtype == FDMLA_BF16 && d % 8 == 0 && k <= 32 &&
                        (((uintptr_t)y | (uintptr_t)out | (uintptr_t)shared) % 16) == 0;
    if (vec_ok)
        combine_bf16x8_kernel<<<T, d >= 2048 ? 256 : 128, 0, s>>>(static_cast<const __nv_bfloat16 *>(y), pos, w,
                                                                  static_cast<const __nv_bfloat16 *>(shared),
                                                                  static_cast<__nv_bfloat16 *>(out), T, k, d);
    else if (dtype == FDMLA_BF16)
        combine_kernel<__nv_bfloat16><<<T, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(y), pos, w,
                                                        static_cast<const __nv_bfloat16 *>(shared),
                                                        static_cast<__nv_bfloat16 *>(out), T, k, d);
    else
        combine_kernel<float><<<T, 256, 0, s>>>(static_cast<const float *>(y), pos, w, static_cast<const float *>(shared),
                                                static_cast<float *>(out), T, k, d);
    return launch_ok();
}
