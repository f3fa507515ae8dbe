// Tensor-core (tcgen05) latent projections and their weight gradient for the on-the-fly
// DMLA mode (bf16, widths 64 and 128), sm_100a.
//
//   project:  Y[rows, d_out] = X[rows, d_in] W        (W [d_in, d_out])   K_lat = K WK
//             Y[rows, d_out] = X[rows, d_in] W^T      (W [d_out, d_in])   dK = dK_lat WK^T
//             X bf16 or fp32 (the latent gradients are kept in fp32), Y bf16, fp32 accumulation
//   wgrad:    P[d_in, d_out] = sum over a run of rows of X[r, :]^T G[r, :]   (X bf16, G fp32),
//             one fp32 partial per CTA, summed in a fixed order by the caller
// These are thin, memory-bound GEMMs (43 FLOP per byte), so each 128-row tile is one CTA:
// operands are read with plain coalesced loads, converted to bf16 and laid out in shared
// memory in the 128-byte swizzle the MMA descriptors expect (K-major for X in `project`,
// MN-major - reduction over the tile's rows - for both operands of `wgrad`), one thread
// issues the K/16 MMAs of the tile, and thread = output row for the epilogue.  Several
// CTAs per SM hide the latencies.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "ptx.cuh"

namespace fdmla {
namespace tcp {

constexpr int TILE = 128;
constexpr int CHUNK = TILE * 128;      // one 64-column chunk of a 128-row tile: 16 384 B

// element (row r, column c) of a [rows x cols] bf16 tile stored as 64-column chunks of
// [rows x 128 B] in the 128-byte swizzle; `rows` is the tile height
__device__ __forceinline__ uint32_t sw_off(int r, int c, int rows) {
    return (uint32_t)((c >> 6) * rows * 128 + r * 128 + ((((c & 63) >> 3) ^ (r & 7)) << 4) + ((c & 7) << 1));
}

// Stores 8 consecutive elements (columns c .. c+7, c % 8 == 0) of row r.
__device__ __forceinline__ void put8(uint8_t *tile, int r, int c, int rows, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
        w[e] = *reinterpret_cast<uint32_t *>(&h);
    }
    *reinterpret_cast<uint4 *>(tile + sw_off(r, c, rows)) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162 *>(&w[e]);
        v[2 * e] = __low2float(h);
        v[2 * e + 1] = __high2float(h);
    }
}

// [n_rows x n_cols] row-major global matrix (rows beyond `valid_rows` read as zero) -> swizzled tile
template <typename T>
__device__ __forceinline__ void stage_tile(uint8_t *tile, const T *src, int n_rows, int n_cols, long long valid_rows) {
    const int vec_per_row = n_cols >> 3;
    for (int idx = threadIdx.x; idx < n_rows * vec_per_row; idx += blockDim.x) {
        const int r = idx / vec_per_row, c = (idx - r * vec_per_row) << 3;
        float v[8];
        if (r < valid_rows) load8<T>(src + (size_t)r * n_cols + c, v);
        else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        }
        put8(tile, r, c, n_rows, v);
    }
}

// ---------------------------------------------------------------------------------------
// project: one CTA per 128-row tile.  WT = 0: W [DIN, DOUT] (B operand MN-major, reduction over
// its rows); WT = 1: W [DOUT, DIN] (B operand K-major).
// ---------------------------------------------------------------------------------------
template <typename TX, int DIN, int DOUT, int WT>
__global__ void __launch_bounds__(128, 3)
project_tc_kernel(const TX *__restrict__ X, const __nv_bfloat16 *__restrict__ W, __nv_bfloat16 *__restrict__ Y, long long rows) {
    using namespace ptx;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sX = smem;                                   // [128 x DIN], K-major
    uint8_t *sW = sX + TILE * DIN * 2;                    // WT = 0: [DIN x DOUT]; WT = 1: [DOUT x DIN]
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    const long long r0 = (long long)blockIdx.x * TILE;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); fence_mbar_init(); }
    if (warp == 0) { tmem_alloc(smem_u32(&tmem_slot), 128); tmem_relinquish(); }
    stage_tile<TX>(sX, X + (size_t)r0 * DIN, TILE, DIN, rows - r0);
    if (WT == 0) stage_tile<__nv_bfloat16>(sW, W, DIN, DOUT, DIN);
    else stage_tile<__nv_bfloat16>(sW, W, DOUT, DIN, DOUT);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = make_idesc_bf16(128, DOUT, 0, WT == 0 ? 1 : 0);
#pragma unroll
        for (int k = 0; k < DIN / 16; ++k) {
            // X: K-major, 64-column chunks of [128 x 128 B]
            const uint64_t da = make_smem_desc(smem_u32(sX) + (k >> 2) * CHUNK + (k & 3) * 32, 16, 1024, kLayoutSw128);
            uint64_t db;
            if (WT == 0)   // rows of the tile are the reduction index: 16 rows per step, chunks of 64 output columns
                db = make_smem_desc(smem_u32(sW) + k * 2048, DIN * 128, 1024, kLayoutSw128);
            else           // rows are output columns, 64-column chunks along the reduction
                db = make_smem_desc(smem_u32(sW) + (k >> 2) * (DOUT * 128) + (k & 3) * 32, 16, 1024, kLayoutSw128);
            mma_bf16_ss(tmem, da, db, idesc, k != 0);
        }
        mma_commit(smem_u32(&bar));
    }
    const bool ok = mbar_wait(smem_u32(&bar), 0);
    tc_fence_after_sync();
    const long long row = r0 + threadIdx.x;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll 1
    for (int cc = 0; cc < DOUT / 32; ++cc) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_base + cc * 32, o);
        tmem_wait_ld();
        if (row < rows && ok) {
            __nv_bfloat16 *dst = Y + (size_t)row * DOUT + cc * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 16) {
                uint32_t w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[j + 2 * e]), __uint_as_float(o[j + 2 * e + 1]));
                    w[e] = *reinterpret_cast<uint32_t *>(&h);
                }
                st_global_v8(dst + j, w);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem, 128); }
}

// ---------------------------------------------------------------------------------------
// wgrad partial: CTA b sums X^T G over the 128-row tiles [b * per, (b + 1) * per) into part[b].
// A = X tile as [rows x 128] (MN-major: M = the 128 columns of X), B = G tile [rows x 64]
// (MN-major), reduction over the tile's rows.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 3)
wgrad_tc_kernel(const __nv_bfloat16 *__restrict__ X, const float *__restrict__ G, float *__restrict__ part, long long rows,
                int tiles_per_cta) {
    using namespace ptx;
    constexpr int DIN = 128, DOUT = 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sX = smem;                    // [128 rows x 128 cols]
    uint8_t *sG = sX + TILE * DIN * 2;     // [128 rows x 64 cols]
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); fence_mbar_init(); }
    if (warp == 0) { tmem_alloc(smem_u32(&tmem_slot), 64); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const long long n_tiles = (rows + TILE - 1) / TILE;
    const long long t_begin = (long long)blockIdx.x * tiles_per_cta;
    long long t_end = t_begin + tiles_per_cta;
    if (t_end > n_tiles) t_end = n_tiles;
    bool ok = true;
    int it = 0;
    for (long long t = t_begin; t < t_end; ++t, ++it) {
        const long long r0 = t * TILE;
        if (it > 0) {
            ok = ok && mbar_wait(smem_u32(&bar), (it - 1) & 1);     // the previous tile's MMAs have read shared memory
            __syncthreads();
        }
        stage_tile<__nv_bfloat16>(sX, X + (size_t)r0 * DIN, TILE, DIN, rows - r0);
        stage_tile<float>(sG, G + (size_t)r0 * DOUT, TILE, DOUT, rows - r0);
        fence_proxy_async_smem();
        __syncthreads();
        tc_fence_after_sync();
        if (threadIdx.x == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(128, DOUT, 1, 1);
#pragma unroll
            for (int k = 0; k < TILE / 16; ++k) {
                const uint64_t da = make_smem_desc(smem_u32(sX) + k * 2048, CHUNK, 1024, kLayoutSw128);
                const uint64_t db = make_smem_desc(smem_u32(sG) + k * 2048, CHUNK, 1024, kLayoutSw128);
                mma_bf16_ss(tmem, da, db, idesc, (it | k) != 0);
            }
            mma_commit(smem_u32(&bar));
        }
    }
    if (it > 0) ok = ok && mbar_wait(smem_u32(&bar), (it - 1) & 1);
    tc_fence_after_sync();
    // thread m holds row m of the [128 x 64] partial
    float *dst = part + (size_t)blockIdx.x * DIN * DOUT + (size_t)threadIdx.x * DOUT;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll 1
    for (int cc = 0; cc < DOUT / 32; ++cc) {
        uint32_t o[32];
        if (it > 0) {
            tmem_ld32(tmem + lane_base + cc * 32, o);
            tmem_wait_ld();
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4 *>(dst + cc * 32 + j) =
                (it > 0 && ok) ? make_float4(__uint_as_float(o[j]), __uint_as_float(o[j + 1]), __uint_as_float(o[j + 2]), __uint_as_float(o[j + 3]))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem, 64); }
}

template <typename TX, int DIN, int DOUT, int WT>
static int launch_project_one(const void *X, const void *W, void *Y, long long rows, cudaStream_t stream) {
    constexpr int smem = 1024 + TILE * DIN * 2 + DIN * DOUT * 2;
    auto kern = project_tc_kernel<TX, DIN, DOUT, WT>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FDMLA_ERR_CUDA;
    const long long blocks = (rows + TILE - 1) / TILE;
    if (blocks > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    kern<<<(unsigned)blocks, 128, smem, stream>>>(static_cast<const TX *>(X), static_cast<const __nv_bfloat16 *>(W),
                                                 static_cast<__nv_bfloat16 *>(Y), rows);
    return check_launch();
}

}  // namespace tcp

// Returns FDMLA_ERR_UNSUPPORTED when the shape is not one of the tensor-core cases (the caller then
// uses the CUDA-core kernel).
int launch_project_tensor(const void *X, const void *W, void *Y, long long rows, int d_in, int d_out, int w_transposed,
                          int x_f32, cudaStream_t stream) {
    using bf = __nv_bfloat16;
    const uintptr_t a = reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y);
    if (a & 31) return FDMLA_ERR_UNSUPPORTED;
    if (d_in == 128 && d_out == 64 && !w_transposed)
        return x_f32 ? tcp::launch_project_one<float, 128, 64, 0>(X, W, Y, rows, stream)
                     : tcp::launch_project_one<bf, 128, 64, 0>(X, W, Y, rows, stream);
    if (d_in == 64 && d_out == 128 && w_transposed)
        return x_f32 ? tcp::launch_project_one<float, 64, 128, 1>(X, W, Y, rows, stream)
                     : tcp::launch_project_one<bf, 64, 128, 1>(X, W, Y, rows, stream);
    return FDMLA_ERR_UNSUPPORTED;
}

// part[n_part][128 * 64] fp32; CTA b covers a contiguous run of 128-row tiles.
int launch_wgrad_partial_tensor(const void *X, const float *G, float *part, long long rows, int d_in, int d_out, int n_part,
                                cudaStream_t stream) {
    if (d_in != 128 || d_out != 64 || n_part <= 0) return FDMLA_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(G) | reinterpret_cast<uintptr_t>(part)) & 15) return FDMLA_ERR_UNSUPPORTED;
    const long long n_tiles = (rows + tcp::TILE - 1) / tcp::TILE;
    const int per = (int)((n_tiles + n_part - 1) / n_part);
    constexpr int smem = 1024 + tcp::TILE * 128 * 2 + tcp::TILE * 64 * 2;
    if (cudaFuncSetAttribute(tcp::wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FDMLA_ERR_CUDA;
    tcp::wgrad_tc_kernel<<<n_part, 128, smem, stream>>>(static_cast<const __nv_bfloat16 *>(X), G, part, rows, per);
    return check_launch();
}

}  // namespace fdmla
