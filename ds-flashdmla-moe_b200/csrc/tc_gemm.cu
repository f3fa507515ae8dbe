// Batched bf16 GEMM on the sm_100a tensor cores (tcgen05 + TMA), for the GEMMs that sit either side of the
// attention kernel and inside the MoE layer:
//   * the absorbed query projection  Q'[n, h, :512] = q_nope[n, h, :] W_UK[h]^T     (batch = heads, B K-major)
//   * the absorbed output projection o[n, h, :]     = O_lat[n, h, :] W_UV[h]       (batch = heads, B MN-major)
//   * the expert MLPs of a MoE layer over padded packing: [E, capacity, d] x [E, d, d_ff] with the SwiGLU gate
//     fused into the epilogue, and [E, capacity, d_ff] x [E, d_ff, d]            (batch = experts, B MN-major)
// (README.md:16-20 of the reference names these steps; it ships no source for them.)
//
// C[b] (M x N) = A[b] (M x K) * B[b], fp32 accumulation, bf16 in and out.  Every operand is a window of a 2-D
// row-major bf16 tensor: batch b of A starts at row b * a_brow, column b * a_bcol of its tensor (so a batch can run
// down the rows - experts - or across the columns - heads of a [tokens, heads * width] activation), likewise B and C.
// B is either K-major ([N, K] rows, the reduction index contiguous) or MN-major ([K, N] rows, the output column
// contiguous).  Gated mode: the accumulator of a tile holds 128 columns of A*B next to the same 128 columns of A*B2
// and the epilogue writes silu(A*B) .* (A*B2) (one [M x 128] tile of C).
//
// Persistent grid, one CTA per SM, 128 x 256 accumulator tiles (two of them in tensor memory, so the epilogue of one
// tile runs under the main loop of the next), K in steps of 64 through a ring of four 48 KB stages filled by TMA in
// the 128-byte swizzle.  Warp 0 issues the copies, warp 1 the MMAs (one elected lane of a converged warp each),
// warps 2-5 read the accumulator (thread = row) and store bf16 rows.  Every wait is bounded; a wait that gives up
// sets a flag that fdmla_device_error_flag reports (code 21-23) and the roles run out.
//
// Problems whose batch entries fill 256-row tiles as well as 128-row ones run the same kernel over CTA pairs (clusters of two,
// tcgen05.mma.cta_group::2): a tile is 256 x 256, each CTA loads its 128 rows of A and HALF of the B tile (128
// output columns) and holds its 128 rows of the accumulator, so a k step costs 32 KB of shared memory per CTA
// instead of 48 KB (six stages) and B crosses L2 -> shared memory once per pair.  Both CTAs' copies signal the
// leader's "full" barrier directly (cta_group::2 loads, no multicast); the leader's warp 1 issues the pair's MMAs
// and its commits arrive on the "empty" / "accumulator full" barriers of both CTAs.  In gated mode the leader's
// half of the B tile is B and the peer's is B2.  FDMLA_GEMM_PAIR=0 / 1 in the environment forces one form.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace fdmla {

bool make_tensor_map_bf16(CUtensorMap *m, const void *base, long long rows, int cols, int box_rows);
bool make_tensor_map_bf16_chunked(CUtensorMap *m, const void *base, long long rows, int cols, int box_rows, int box_chunks);

namespace tcg {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2;          // 16 384: the 128 rows of A one CTA loads per k step
constexpr int THREADS = 192;
template <bool PAIR> struct Cfg {
    static constexpr int TILE_M = PAIR ? 2 * BM : BM;             // rows of one accumulator tile (both CTAs of a pair)
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2; // of one CTA: 16 384 / 32 768
    static constexpr int STAGES = PAIR ? 6 : 4;
    static constexpr int STAGE = A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE + 256;
    static_assert(SMEM_BYTES <= kMaxSmemPerBlock, "shared memory overflow");
    static_assert((2 * STAGES + 4) * 8 + 8 <= 256, "barriers overflow their space");
};
enum { ERR_PRODUCER = 21, ERR_MMA = 22, ERR_EPILOGUE = 23 };

__device__ int g_gemm_error = 0;

struct Problem {
    int batch, M, N, K;                 // N: output columns per batch entry
    int a_brow, a_bcol;                 // window of batch b in A's tensor: row b * a_brow, column b * a_bcol
    int b_brow, b_bcol;                 // K-major: rows are output columns; MN-major: rows are the reduction index
    long long c_brow, c_bcol, ldc;      // C element (b, m, n) = C[(b * c_brow + m) * ldc + b * c_bcol + n]
    void *C;                            // bf16, or fp32 when c_f32
    int b_k_major, gated;
    int c_f32, accumulate;              // fp32 output; accumulate (fp32 only): C += alpha A B instead of C = alpha A B
    float alpha;
    int m_tiles, n_tiles;
    // Grouped (ragged) mode: batch entry b owns rows [row_offsets[b], row_offsets[b + 1]) of A's and C's tensors (read on the
    // device: the packed rows of a MoE layer, whose per-expert counts the host never sees); M is then only an upper bound.
    const int32_t *row_offsets;
    // Causal hint (attention backward; 0 = none).  Row m of an entry is query position (causal_row0 + m) mod
    // causal_period and sees columns / reduction indices <= position + causal_off.
    //   1: output tiles whose columns no row of the tile sees are not computed and not written (S, dP: the consumer
    //      does not read them);  2: the reduction of a tile stops behind the last index one of its rows sees (dQ = dS K:
    //      dS is zero beyond it).
    int causal_mode, causal_period, causal_off, causal_row0;
};

// last column / reduction index that a row of the tile [m0, m0 + tile_m) sees (a tile that runs over the end of a period
// sees everything the period's last position sees)
__device__ __forceinline__ int causal_limit(const Problem &p, int m0, int tile_m) {
    const int q0 = (p.causal_row0 + m0) % p.causal_period;
    const int q1 = q0 + tile_m - 1;
    return (q1 >= p.causal_period ? p.causal_period - 1 : q1) + p.causal_off;
}
__device__ __forceinline__ bool tile_skipped(const Problem &p, int m0, int n0, int tile_m) {
    return p.causal_mode == 1 && n0 > causal_limit(p, m0, tile_m);
}
__device__ __forceinline__ int tile_k_steps(const Problem &p, int m0, int tile_m, int k_steps) {
    if (p.causal_mode != 2) return k_steps;
    const int need = (causal_limit(p, m0, tile_m) + BK) / BK;        // indices 0 .. limit
    return need < 1 ? 1 : (need < k_steps ? need : k_steps);
}

// Walks the tiles of a launch in increasing order: tile -> (batch entry, first row, first column, rows of the entry).
struct TileWalker {
    int b = 0;
    long long base = 0;          // tiles of the entries before b
    int m0, n0, rows, row0;      // of the located tile: first row inside the entry, first output column, the entry's rows
                                 // and its first row in A's / C's tensor (grouped mode)
    __device__ __forceinline__ bool locate(const Problem &p, long long tile, int out_cols, int tile_m) {
        if (!p.row_offsets) {
            const int per = p.m_tiles * p.n_tiles;
            if (tile >= (long long)p.batch * per) return false;
            b = (int)(tile / per);
            const int r = (int)(tile - (long long)b * per);
            n0 = (r / p.m_tiles) * out_cols;
            m0 = (r % p.m_tiles) * tile_m;
            rows = p.M;
            row0 = 0;
            return true;
        }
        while (b < p.batch) {
            const int lo = __ldg(p.row_offsets + b), hi = __ldg(p.row_offsets + b + 1);
            const int mt = (hi - lo + tile_m - 1) / tile_m;
            const long long tb = (long long)(mt > 0 ? mt : 0) * p.n_tiles;
            if (tile < base + tb) {
                const int r = (int)(tile - base);
                n0 = (r / mt) * out_cols;
                m0 = (r % mt) * tile_m;
                rows = hi - lo;
                row0 = lo;
                return true;
            }
            base += tb;
            ++b;
        }
        return false;
    }
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

template <bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const Problem p, const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmB2) {
    using namespace ptx;
    using C = Cfg<PAIR>;
    constexpr int STAGES = C::STAGES, STAGE = C::STAGE, B_BYTES = C::B_BYTES, TILE_M = C::TILE_M;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    int *err_slot = reinterpret_cast<int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto FULL = [&](int s) { return bar0 + 8u * s; };
    auto EMPTY = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto ACC_FULL = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto ACC_EMPTY = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // pair form: CTA `rank` of the cluster owns rows [128 rank, +128) of every tile and half of its B operand
    const int rank = PAIR ? (int)cluster_ctarank() : 0;
    const long long first_tile = PAIR ? blockIdx.x >> 1 : blockIdx.x;
    const long long tile_step = PAIR ? gridDim.x >> 1 : gridDim.x;

    if (threadIdx.x == 0) {
        *err_slot = *reinterpret_cast<volatile int *>(&g_gemm_error);      // one reading for all roles
        for (int s = 0; s < STAGES; ++s) { mbar_init(FULL(s), 1); mbar_init(EMPTY(s), 1); }
        // accumulator free: every epilogue thread arrives; pair form: one arrival per CTA, on the leader's barrier
        for (int a = 0; a < 2; ++a) { mbar_init(ACC_FULL(a), 1); mbar_init(ACC_EMPTY(a), PAIR ? 2 : 128); }
        fence_mbar_init();
    }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_2cta(smem_u32(tmem_slot), 512); tmem_relinquish_2cta(); }
        else { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) { __syncwarp(); cluster_sync_all(); }      // the peer's barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // an earlier launch gave up a wait: do nothing until the flag is cleared (both CTAs of a pair take the leader's reading)
    const bool poisoned = (PAIR ? (int)ld_shared_cluster_u32(map_to_cta(smem_u32(err_slot), 0)) : *err_slot) != 0;

    const int k_steps = p.K / BK;
    const int out_cols = p.gated ? BN / 2 : BN;         // output columns of one tile
    // tile -> (batch entry, m tile, n tile): the m tiles of one (entry, n tile) are neighbours, so CTAs that run at the
    // same time share the B tile in L2.  Every role walks the same tiles with its own TileWalker.

    if (warp == 0) {
        // ================================ TMA producer ================================
        const bool elected = elect_one();
        if (lane == 0) { prefetch_tmap(&tmA); prefetch_tmap(&tmB); if (p.gated) prefetch_tmap(&tmB2); }
        const uint32_t full_lead = PAIR ? map_to_cta(FULL(0), 0) : 0;     // the leader's "full" barriers
        bool ok = true;
        int s = 0, use = 0;
        TileWalker w;
        for (long long tile = first_tile; !poisoned && ok && w.locate(p, tile, out_cols, TILE_M); tile += tile_step) {
            const int b = w.b, m0 = w.m0, n0 = w.n0;
            if (tile_skipped(p, m0, n0, TILE_M)) continue;
            const int a_row = (p.row_offsets ? w.row0 : b * p.a_brow) + m0 + rank * BM;
            const int ks = tile_k_steps(p, m0, TILE_M, k_steps);
            for (int kb = 0; kb < ks && ok; ++kb) {
                if (use > 0) ok = mbar_wait(EMPTY(s), (use - 1) & 1);
                if (ok && elected) {
                    const uint32_t dstA = smem_u32(smem + s * STAGE), dstB = dstA + A_BYTES;
                    if constexpr (PAIR) {
                        const uint32_t full = full_lead + 8u * s;
                        if (rank == 0) mbar_arrive_expect_tx(FULL(s), 2 * STAGE);     // both CTAs' bytes
                        tma_load_2d_pair(dstA, &tmA, b * p.a_bcol + kb * BK, a_row, full);
                        // this CTA's half of B: 128 output columns; gated: the leader brings B, the peer B2
                        const CUtensorMap *tb = (p.gated && rank) ? &tmB2 : &tmB;
                        const int n_half = n0 + (p.gated ? 0 : rank * (BN / 2));
                        if (p.b_k_major) tma_load_2d_pair(dstB, tb, b * p.b_bcol + kb * BK, b * p.b_brow + n_half, full);
                        else tma_load_3d_pair(dstB, tb, 0, b * p.b_brow + kb * BK, (b * p.b_bcol + n_half) >> 6, full);
                    } else {
                        mbar_arrive_expect_tx(FULL(s), STAGE);
                        tma_load_2d(dstA, &tmA, b * p.a_bcol + kb * BK, a_row, FULL(s));
                        if (p.b_k_major) {
                            // [256 output columns x 64] K-major: rows of B's tensor are output columns
                            tma_load_2d(dstB, &tmB, b * p.b_bcol + kb * BK, b * p.b_brow + n0, FULL(s));
                            if (p.gated) tma_load_2d(dstB + B_BYTES / 2, &tmB2, b * p.b_bcol + kb * BK, b * p.b_brow + n0, FULL(s));
                        } else {
                            // [64 x 256 output columns] MN-major: four (gated: two and two) chunks of [64 rows x 128 B]
                            const int chunk0 = (b * p.b_bcol + n0) >> 6;
                            tma_load_3d(dstB, &tmB, 0, b * p.b_brow + kb * BK, chunk0, FULL(s));
                            if (p.gated) tma_load_3d(dstB + B_BYTES / 2, &tmB2, 0, b * p.b_brow + kb * BK, chunk0, FULL(s));
                        }
                    }
                }
                if (++s == STAGES) { s = 0; ++use; }
            }
        }
        if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, ERR_PRODUCER);
        __syncwarp();
    } else if (warp == 1) {
        // ================================ MMA issuer (pair form: the leader's only) ==================================
        const bool elected = elect_one();
        const uint32_t idesc = make_idesc_bf16(TILE_M, BN, 0, p.b_k_major ? 0 : 1);
        bool ok = true;
        int s = 0;
        uint32_t ph = 0;
        int n_done = 0;                              // tiles this CTA has issued
        TileWalker w;
        for (long long tile = first_tile; !poisoned && rank == 0 && w.locate(p, tile, out_cols, TILE_M); tile += tile_step) {
            if (!__all_sync(0xffffffffu, ok)) break;
            if (tile_skipped(p, w.m0, w.n0, TILE_M)) continue;
            const int ks = tile_k_steps(p, w.m0, TILE_M, k_steps);
            const int acc = n_done & 1;
            if (n_done >= 2) {
                ok = ok && mbar_wait(ACC_EMPTY(acc), ((n_done >> 1) - 1) & 1);     // the epilogue has read this accumulator
                tc_fence_after_sync();
            }
            for (int kb = 0; kb < ks; ++kb) {
                ok = ok && mbar_wait(FULL(s), ph);
                tc_fence_after_sync();
                if (elected) {
                    const uint32_t a_addr = smem_u32(smem + s * STAGE), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = make_smem_desc(a_addr + k * 32, 16, 1024, kLayoutSw128);
                        const uint64_t db = p.b_k_major ? make_smem_desc(b_addr + k * 32, 16, 1024, kLayoutSw128)
                                                        : make_smem_desc(b_addr + k * 2048, 8192, 1024, kLayoutSw128);
                        if constexpr (PAIR) mma_bf16_ss_2cta(tmem + acc * BN, da, db, idesc, (kb | k) != 0);
                        else mma_bf16_ss(tmem + acc * BN, da, db, idesc, (kb | k) != 0);
                    }
                    if constexpr (PAIR) {
                        mma_commit_2cta(EMPTY(s), 3);
                        if (kb == ks - 1) mma_commit_2cta(ACC_FULL(acc), 3);
                    } else {
                        mma_commit(EMPTY(s));
                        if (kb == ks - 1) mma_commit(ACC_FULL(acc));
                    }
                }
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            ++n_done;
        }
        if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, ERR_MMA);
        __syncwarp();
    } else {
        // ================================ epilogue ====================================
        const int L = (warp & 3) * 32 + lane;                      // TMEM lane = row of this CTA's part of the tile
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t acc_empty_lead = PAIR ? map_to_cta(ACC_EMPTY(0), 0) : 0;
        bool ok = true;
        int n_done = 0;
        TileWalker w;
        for (long long tile = first_tile; !poisoned && w.locate(p, tile, out_cols, TILE_M); tile += tile_step) {
            const int b = w.b, m0 = w.m0, n0 = w.n0;
            if (tile_skipped(p, m0, n0, TILE_M)) continue;
            const int acc = n_done & 1;
            if (ok) ok = mbar_wait(ACC_FULL(acc), (n_done >> 1) & 1);
            tc_fence_after_sync();
            const int m = m0 + rank * BM + L;
            const long long c_off = ((p.row_offsets ? (long long)w.row0 : (long long)b * p.c_brow) + m) * p.ldc +
                                    (long long)b * p.c_bcol + n0;
            __nv_bfloat16 *crow = static_cast<__nv_bfloat16 *>(p.C) + c_off;
            float *crow_f = static_cast<float *>(p.C) + c_off;
            const uint32_t t0 = tmem + lane_base + acc * BN;
#pragma unroll 1
            for (int c = 0; c < out_cols / 32; ++c) {
                uint32_t r[32], g[32];
                if (ok) {
                    tmem_ld32(t0 + c * 32, r);
                    if (p.gated) tmem_ld32(t0 + BN / 2 + c * 32, g);
                    tmem_wait_ld();
                }
                if (!ok || m >= w.rows || n0 + c * 32 >= p.N) continue;
                if (p.c_f32) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint32_t w8[8];
                        float4 o0 = make_float4(0.f, 0.f, 0.f, 0.f), o1 = o0;
                        if (p.accumulate) {
                            o0 = *reinterpret_cast<const float4 *>(crow_f + c * 32 + j);
                            o1 = *reinterpret_cast<const float4 *>(crow_f + c * 32 + j + 4);
                        }
                        const float old[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                        for (int e = 0; e < 8; ++e) w8[e] = __float_as_uint(fmaf(p.alpha, __uint_as_float(r[j + e]), old[e]));
                        st_global_v8(crow_f + c * 32 + j, w8);
                    }
                    continue;
                }
#pragma unroll
                for (int j = 0; j < 32; j += 16) {
                    uint32_t w[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float x0 = __uint_as_float(r[j + 2 * e]) * p.alpha, x1 = __uint_as_float(r[j + 2 * e + 1]) * p.alpha;
                        if (p.gated) {
                            x0 = silu(x0) * __uint_as_float(g[j + 2 * e]);
                            x1 = silu(x1) * __uint_as_float(g[j + 2 * e + 1]);
                        }
                        __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
                        w[e] = *reinterpret_cast<uint32_t *>(&h);
                    }
                    st_global_v8(crow + c * 32 + j, w);
                }
            }
            tc_fence_before_sync();
            if constexpr (PAIR) {
                named_bar_sync(1, 128);                                // this CTA's 128 rows have been read ...
                if (L == 0) mbar_arrive_cluster_relaxed(acc_empty_lead + 8u * acc);   // ... one arrival per CTA frees the accumulator
            } else {
                mbar_arrive(ACC_EMPTY(acc));                           // 128 arrivals free the accumulator
            }
            ++n_done;
        }
        if (!ok) atomicCAS(&g_gemm_error, 0, ERR_EPILOGUE);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) { __syncwarp(); cluster_sync_all(); }      // neither CTA leaves while the pair can still touch its memory
    if (warp == 1) {
        tc_fence_after_sync();
        if (PAIR) tmem_dealloc_2cta(tmem, 512); else tmem_dealloc(tmem, 512);
    }
}

// CTA pairs that can be resident at once (cached per device); 0 if clusters of two cannot be launched
static int max_pairs(int dev, int sms) {
    static std::atomic<int> cached[64];
    if (dev < 0 || dev >= 64) return sms / 2;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n != 0) return n > 0 ? n : 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (unsigned)(sms / 2));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true>::SMEM_BYTES) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, gemm_kernel<true>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = -1;
    }
    cached[dev].store(n, std::memory_order_relaxed);
    return n > 0 ? n : 0;
}

}  // namespace tcg

int gemm_error_flag(int reset) {
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, tcg::g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(tcg::g_gemm_error, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return v;
}

// Arguments as in fdmla_gemm_batched (include/flashdmla.h); with row_offsets (fdmla_gemm_grouped) M is the total number
// of rows and batch entry b owns rows [row_offsets[b], row_offsets[b + 1]) of A and C.
int launch_gemm_batched(const void *A, const void *B, const void *B2, void *C, int batch, int M, int N, int K,
                        long long a_rows, long long lda, int a_brow, int a_bcol, long long b_rows, long long ldb,
                        int b_brow, int b_bcol, int b_k_major, long long ldc, long long c_brow, long long c_bcol,
                        int gated, const int32_t *row_offsets, cudaStream_t stream, float alpha, int c_f32, int accumulate,
                        const GemmCausalHint *causal) {
    using namespace tcg;
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return FDMLA_OK;
    if (K % BK != 0 || N % 64 != 0 || lda % 8 != 0 || ldb % 64 != 0 || ldc % (c_f32 ? 8 : 16) != 0) return FDMLA_ERR_UNSUPPORTED;
    if ((accumulate && !c_f32) || (gated && c_f32)) return FDMLA_ERR_UNSUPPORTED;
    if (a_bcol % 8 != 0 || b_bcol % 64 != 0 || c_bcol % 16 != 0) return FDMLA_ERR_UNSUPPORTED;
    if (gated && (N % 128 != 0 || !B2)) return FDMLA_ERR_UNSUPPORTED;
    if (lda > 2147483647LL || ldb > 2147483647LL || a_rows > 2147483647LL || b_rows > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(B2)) & 15) return FDMLA_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(C) & 31) return FDMLA_ERR_UNSUPPORTED;
    Problem p{};
    p.batch = batch; p.M = M; p.N = N; p.K = K;
    p.a_brow = a_brow; p.a_bcol = a_bcol; p.b_brow = b_brow; p.b_bcol = b_bcol;
    p.c_brow = c_brow; p.c_bcol = c_bcol; p.ldc = ldc; p.C = C;
    p.alpha = alpha; p.c_f32 = c_f32 ? 1 : 0; p.accumulate = accumulate ? 1 : 0;
    p.b_k_major = b_k_major ? 1 : 0; p.gated = gated ? 1 : 0;
    p.row_offsets = row_offsets;
    if (causal && causal->mode != 0) {
        if (row_offsets || causal->period <= 0 || causal->mode < 0 || causal->mode > 2 || (accumulate && causal->mode == 1))
            return FDMLA_ERR_INVALID;
        p.causal_mode = causal->mode; p.causal_period = causal->period; p.causal_off = causal->off;
        p.causal_row0 = (int)(causal->row0 % causal->period);
    }
    int dev = 0, sms = kNumSMs;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // CTA pairs with 256-row tiles when that pads an entry's rows no further than 128-row tiles would (ragged entries:
    // when they are tall enough for the half tile more that each may waste not to matter)
    static const int forced = [] { const char *e = getenv("FDMLA_GEMM_PAIR"); return e && *e ? atoi(e) : -1; }();
    bool pair = row_offsets ? (long long)M >= 512LL * batch : (M > BM && ((M + BM - 1) / BM) % 2 == 0);
    if (forced >= 0) pair = forced != 0;
    const int pairs = pair ? max_pairs(dev, sms) : 0;
    if (pairs <= 0) pair = false;
    const int tile_m = pair ? 2 * BM : BM;
    const int out_cols = gated ? BN / 2 : BN;
    p.m_tiles = (M + tile_m - 1) / tile_m;
    p.n_tiles = (N + out_cols - 1) / out_cols;
    CUtensorMap tmA, tmB, tmB2;
    if (!make_tensor_map_bf16(&tmA, A, a_rows, (int)lda, BM)) return FDMLA_ERR_CUDA;
    // output columns brought by one copy: a CTA of a pair brings 128 (all of its half: B, or B2 in the peer when gated)
    const int b_box = (gated || pair) ? BN / 2 : BN;
    if (b_k_major) {
        if (!make_tensor_map_bf16(&tmB, B, b_rows, (int)ldb, b_box)) return FDMLA_ERR_CUDA;
        tmB2 = tmB;
        if (gated && !make_tensor_map_bf16(&tmB2, B2, b_rows, (int)ldb, b_box)) return FDMLA_ERR_CUDA;
    } else {
        if (!make_tensor_map_bf16_chunked(&tmB, B, b_rows, (int)ldb, BK, b_box / 64)) return FDMLA_ERR_CUDA;
        tmB2 = tmB;
        if (gated && !make_tensor_map_bf16_chunked(&tmB2, B2, b_rows, (int)ldb, BK, b_box / 64)) return FDMLA_ERR_CUDA;
    }
    // grouped mode: M is the total of all entries' rows; every entry may add one partly filled row tile
    const long long tiles = row_offsets ? ((long long)(M + tile_m - 1) / tile_m + batch) * p.n_tiles : (long long)batch * p.m_tiles * p.n_tiles;
    if (pair) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (unsigned)(tiles < pairs ? tiles : pairs));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
        cfg.attrs = &at;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, gemm_kernel<true>, p, tmA, tmB, tmB2) != cudaSuccess) { cudaGetLastError(); return FDMLA_ERR_CUDA; }
        return check_launch();
    }
    if (cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false>::SMEM_BYTES) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    const int grid = (int)(tiles < sms ? tiles : sms);
    gemm_kernel<false><<<grid, THREADS, Cfg<false>::SMEM_BYTES, stream>>>(p, tmA, tmB, tmB2);
    return check_launch();
}

// y[r, 0:d] = rotary(x[r, 0:d], pos[r / rows_per_pos]) on pairs (2i, 2i+1) with angle pos * base^(-2i/d); x and y are
// rows of wider tensors (row strides ldx, ldy elements).  The 64-wide RoPE tail of the absorbed query: read from the
// per-head query, written next to the 512 latent columns the GEMM above produced.
__global__ void rope_rows_kernel(const __nv_bfloat16 *__restrict__ x, long long ldx, __nv_bfloat16 *__restrict__ y, long long ldy,
                                 const int32_t *__restrict__ pos, long long rows, int rows_per_pos, int d, float log2_base) {
    const int half = d >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * half) return;
    const long long r = idx / half;
    const int i = (int)(idx - r * half);
    const float inv = exp2f(-log2_base * (2.f * i) / d);
    float sn, cs;
    sincosf((float)pos[r / rows_per_pos] * inv, &sn, &cs);
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162 *>(x + r * ldx + 2 * i);
    const float x0 = __low2float(v), x1 = __high2float(v);
    *reinterpret_cast<__nv_bfloat162 *>(y + r * ldy + 2 * i) = __floats2bfloat162_rn(x0 * cs - x1 * sn, x0 * sn + x1 * cs);
}

int launch_rope_rows(const void *x, long long ldx, void *y, long long ldy, const int32_t *pos, long long rows,
                     int rows_per_pos, int d, float base, cudaStream_t stream) {
    if (rows <= 0) return FDMLA_OK;
    if (d <= 0 || (d & 1) || rows_per_pos <= 0 || (ldx & 1) || (ldy & 1) || base <= 0.f) return FDMLA_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 3) return FDMLA_ERR_UNSUPPORTED;
    const long long n = rows * (d >> 1);
    const int threads = 256;
    rope_rows_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(x), ldx, static_cast<__nv_bfloat16 *>(y), ldy, pos, rows, rows_per_pos, d, log2f(base));
    return check_launch();
}

}  // namespace fdmla
