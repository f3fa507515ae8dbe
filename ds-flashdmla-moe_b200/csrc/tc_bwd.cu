// Tensor-core (tcgen05) backward of the attention core for 64-wide latents
// (bf16, d_qk = d_v = 64, separate V: the on-the-fly DMLA mode), sm_100a.
//
// The gradient formulas are those the reference intends in
// csrc/attention/fa2_bwd.cu (delta :198-216, dS = P (dP - delta) :234, dK :252-254,
// dV :259-272, dQ :293-309) with the softmax scale applied:
//   P  = exp(scale S - m) / l         S = Q K^T           dP = dO V^T
//   dS = P o (dP - D)                 D = rowsum(dO o O)
//   dV = P^T dO      dK = scale dS^T Q      dQ = scale dS K
// Two owner-computes kernels, no atomics (the reference accumulates with atomicAdd):
//   MODE_DKV  one CTA owns 128 keys of a KV group and streams the 128-row query tiles:
//             T1 = K Q^T (= S^T), T2 = V dO^T (= dP^T), E1 = P^T, E2 = dS^T,
//             dV += E1 dO, dK += E2 Q
//   MODE_DQ   one CTA owns 128 query rows and streams the 128-key tiles:
//             T1 = Q K^T (= S), T2 = dO V^T (= dP), E2 = dS, dQ += E2 K
// Every operand tile is [128 rows x 64 columns] bf16 = 16 KB, loaded by one TMA copy in the
// 128-byte swizzle; the same tile serves as the K-major operand of T1/T2 (reduction over the
// 64 columns) and as the MN-major B operand of the accumulating GEMM (reduction over its 128
// rows).  T1, T2 and the accumulators live in tensor memory; E1/E2 go through shared memory
// as un-swizzled K-major A operands.  Roles: warps 0-3 elementwise (thread = TMEM lane),
// warp 4 TMA + MMA issue (converged, one elected lane).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace fdmla {

bool make_tensor_map_bf16(CUtensorMap *m, const void *base, long long rows, int cols, int box_rows);

namespace tcb {

constexpr int TILE = 128;                 // rows and keys per tile
constexpr int D = 64;                     // latent width
constexpr int OP_BYTES = TILE * D * 2;    // 16 384: one operand tile
constexpr int HALF = 64;                  // streamed indices per pipeline step (half a tile)
constexpr int E_BYTES = TILE * HALF * 2;  // 16 384: one elementwise result of a half tile (A operand, K = 64)
constexpr int E_SBO = (HALF / 8) * 128;   // 1 024: stride between 8-row groups of the un-swizzled layout
constexpr int VEC_BYTES = 2 * 4 * TILE * 4;
// One streamed-tile buffer, one half-tile set of T1/T2 in tensor memory and one of E1/E2 in shared memory, so that TWO
// CTAs share an SM (101 KB of shared memory and 256 tensor-memory columns each): while one CTA's elementwise warps wait
// for their next half tile's score GEMMs - which with single buffers can only start when the previous half has been
// read - the other CTA's are working.  (Everything double-buffered in one CTA per SM measured 8 % slower.)
constexpr bool LEAN = true;
constexpr int N_SBUF = 1;                 // streamed-tile buffers
constexpr int N_HBUF = 1;                 // half-tile buffers of T1/T2 and E1/E2
// barriers
constexpr int B_OWNER = 0, B_FULL = 1, B_EMPTY = 3, B_SREADY = 5, B_PREADY = 7, B_DONE = 9, NBARS = 10;
constexpr int SMEM_BYTES = 1024 + 2 * OP_BYTES + N_SBUF * 2 * OP_BYTES + 2 * N_HBUF * E_BYTES + VEC_BYTES + NBARS * 8 + 16;
static_assert(SMEM_BYTES <= kMaxSmemPerBlock, "shared memory overflow");
static_assert(!LEAN || 2 * (SMEM_BYTES + 1024) <= 233472, "two CTAs do not fit an SM's shared memory");
constexpr int THREADS = 288;              // 8 elementwise warps (two per TMEM lane quarter) + the control warp
constexpr int CTRL_WARP = 8;
// tensor memory columns (T1/T2: N_HBUF 64-column halves each)
constexpr int C_T1 = 0, C_T2 = N_HBUF * HALF, C_ACC1 = 2 * N_HBUF * HALF, C_ACC2 = C_ACC1 + D, TMEM_COLS = LEAN ? 256 : 512;
static_assert(C_ACC2 + D <= TMEM_COLS, "tensor memory overflow");
__device__ __forceinline__ int sbuf_of(int i) { return LEAN ? 0 : (i & 1); }     // streamed tile i -> its buffer
__device__ __forceinline__ int hbuf_of(int h) { return LEAN ? 0 : h; }           // half h -> its T / E buffer
enum { MODE_DKV = 0, MODE_DQ = 1 };
enum { ERR_BWD = 21 };

__device__ int g_bwd_error = 0;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, LEAN ? 2 : 1)
bwd_tc_kernel(const BwdProblem p, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
    using namespace ptx;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sA1 = smem;                      // owner tile 1 (K or Q)
    uint8_t *sA2 = sA1 + OP_BYTES;            // owner tile 2 (V or dO)
    uint8_t *sB = sA2 + OP_BYTES;             // streamed tiles: [buf][B1 | B2]
    uint8_t *sE1 = sB + N_SBUF * 2 * OP_BYTES;   // P^T, one buffer per half-tile buffer (MODE_DKV only)
    uint8_t *sE2 = sE1 + N_HBUF * E_BYTES;       // dS^T / dS
    float *vec = reinterpret_cast<float *>(sE2 + N_HBUF * E_BYTES);    // [buf][m, 1/l, D, last visible key][128]  (MODE_DKV)
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(vec) + VEC_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = blockIdx.y;
    const int own0 = blockIdx.x * TILE;               // first key (MODE_DKV) or first row (MODE_DQ) owned
    const int off = p.Skv - p.Sq;                     // key j is visible to query position i iff j <= i + off
    // streamed tiles: rows for MODE_DKV, keys for MODE_DQ
    const int n_total = MODE == MODE_DKV ? (p.R + TILE - 1) / TILE : (p.Skv + TILE - 1) / TILE;
    int s_first = 0, s_end = n_total;
    if (p.causal) {
        if (MODE == MODE_DKV) {
            // rows that can see key own0: i >= own0 - off; tiles can only be skipped when rows are positions (R == Sq)
            if (p.R == p.Sq) {
                const int i_min = own0 - off;
                s_first = i_min > 0 ? i_min / TILE : 0;
            }
        } else if (p.R == p.Sq) {
            const int r_last = (own0 + TILE - 1 < p.R ? own0 + TILE - 1 : p.R - 1);
            const long long j_max = (long long)r_last + off;         // last visible key of the tile's last row
            if (j_max < 0) s_end = 0;
            else if (j_max / TILE + 1 < s_end) s_end = (int)(j_max / TILE) + 1;
        }
    }
    if (s_first > s_end) s_first = s_end;
    const int n_stream = s_end - s_first;
    const bool poisoned = *reinterpret_cast<volatile int *>(&g_bwd_error) != 0;

    if (threadIdx.x == 0) {
        mbar_init(BAR(B_OWNER), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(BAR(B_FULL + b), 1);
            mbar_init(BAR(B_EMPTY + b), 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(BAR(B_SREADY + h), 1);
            mbar_init(BAR(B_PREADY + h), 1);
        }
        mbar_init(BAR(B_DONE), 1);
        fence_mbar_init();
    }
    if (warp == CTRL_WARP) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const bool active = n_stream > 0 && !poisoned;

    const CUtensorMap *mapA1 = MODE == MODE_DKV ? &tmK : &tmQ, *mapA2 = MODE == MODE_DKV ? &tmV : &tmdO;
    const CUtensorMap *mapB1 = MODE == MODE_DKV ? &tmQ : &tmK, *mapB2 = MODE == MODE_DKV ? &tmdO : &tmV;
    const int own_rows_base = MODE == MODE_DKV ? g * p.Skv : g * p.R;      // global row of the group's first owner row
    const int str_rows_base = MODE == MODE_DKV ? g * p.R : g * p.Skv;

    if (warp == CTRL_WARP) {
        // =========================== TMA + MMA issue ======================================
        if (active) {
            const bool elected = elect_one();
            bool ok = true;
            constexpr uint32_t idesc_t = make_idesc_bf16(128, 128, 0, 0);       // T = A B^T, both K-major
            constexpr uint32_t idesc_acc = make_idesc_bf16(128, 64, 0, 1);      // acc += E B, B MN-major
            auto load_stream = [&](int i) {          // streamed tile i -> its buffer
                const int buf = sbuf_of(i);
                if (elected) {
                    const int row = str_rows_base + (s_first + i) * TILE;
                    mbar_arrive_expect_tx(BAR(B_FULL + buf), 2 * OP_BYTES);
                    tma_load_2d(smem_u32(sB + buf * 2 * OP_BYTES), mapB1, 0, row, BAR(B_FULL + buf));
                    tma_load_2d(smem_u32(sB + buf * 2 * OP_BYTES + OP_BYTES), mapB2, 0, row, BAR(B_FULL + buf));
                }
            };
            if (elected) {
                prefetch_tmap(&tmQ); prefetch_tmap(&tmdO); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
                mbar_arrive_expect_tx(BAR(B_OWNER), 2 * OP_BYTES);
                tma_load_2d(smem_u32(sA1), mapA1, 0, own_rows_base + own0, BAR(B_OWNER));
                tma_load_2d(smem_u32(sA2), mapA2, 0, own_rows_base + own0, BAR(B_OWNER));
            }
            // A streamed tile that runs past the end of its group holds rows of the next group (or the fill value).
            // Their columns of E1 / E2 are zero, but 0 x Inf or 0 x NaN in the accumulating GEMMs is NaN, so those
            // rows are zeroed in shared memory once the copy has landed (whole 128-byte rows: the swizzle does not
            // matter), as the forward kernels do for keys past the end of a sequence.
            auto fix_tail = [&](int i) {
                const int str0 = (s_first + i) * TILE;
                const int limit = MODE == MODE_DKV ? p.R : p.Skv;
                if (str0 + TILE > limit) {
                    const int first_bad = limit > str0 ? limit - str0 : 0;
                    const int n16 = (TILE - first_bad) * 8;
                    uint8_t *b = sB + sbuf_of(i) * 2 * OP_BYTES;
                    for (int idx = lane; idx < 2 * n16; idx += 32) {
                        const int t = idx / n16, rem = idx - t * n16;
                        *reinterpret_cast<uint4 *>(b + t * OP_BYTES + (first_bad + rem / 8) * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                }
            };
            load_stream(0);
            ok = mbar_wait(BAR(B_OWNER), 0);
            constexpr uint32_t idesc_th = make_idesc_bf16(128, HALF, 0, 0);
            // Score GEMMs of one half tile (64 streamed rows): T1[h] = A1 B1[h]^T, T2[h] = A2 B2[h]^T
            auto issue_t = [&](int i, int h) {
                const uint32_t b1 = smem_u32(sB + sbuf_of(i) * 2 * OP_BYTES) + h * (HALF * 128), b2 = b1 + OP_BYTES;
                if (elected) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_bf16_ss(tmem + C_T1 + hbuf_of(h) * HALF, make_smem_desc(smem_u32(sA1) + k * 32, 16, 1024, kLayoutSw128),
                                    make_smem_desc(b1 + k * 32, 16, 1024, kLayoutSw128), idesc_th, k != 0);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_bf16_ss(tmem + C_T2 + hbuf_of(h) * HALF, make_smem_desc(smem_u32(sA2) + k * 32, 16, 1024, kLayoutSw128),
                                    make_smem_desc(b2 + k * 32, 16, 1024, kLayoutSw128), idesc_th, k != 0);
                    mma_commit(BAR(B_SREADY + h));
                }
            };
            // Accumulating GEMMs of one half tile: acc1 += E1[h] B2[h], acc2 += E2[h] B1[h] (reduction over its 64 rows)
            auto issue_acc = [&](int i, int h) {
                const uint32_t b1 = smem_u32(sB + sbuf_of(i) * 2 * OP_BYTES) + h * (HALF * 128), b2 = b1 + OP_BYTES;
                if (elected) {
                    if (MODE == MODE_DKV) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma_bf16_ss(tmem + C_ACC1, make_smem_desc(smem_u32(sE1 + hbuf_of(h) * E_BYTES) + k * 256, 128, E_SBO, kLayoutNone),
                                        make_smem_desc(b2 + k * 2048, OP_BYTES, 1024, kLayoutSw128), idesc_acc, (i | h | k) != 0);
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_bf16_ss(tmem + C_ACC2, make_smem_desc(smem_u32(sE2 + hbuf_of(h) * E_BYTES) + k * 256, 128, E_SBO, kLayoutNone),
                                    make_smem_desc(b1 + k * 2048, OP_BYTES, 1024, kLayoutSw128), idesc_acc, (i | h | k) != 0);
                    if (h == 1) mma_commit(BAR(B_EMPTY + sbuf_of(i)));      // the tile's buffer has been read for the last time
                }
            };
            ok = ok && mbar_wait(BAR(B_FULL), 0);
            fix_tail(0);
            tc_fence_after_sync();
            issue_t(0, 0);
            for (int i = 0; i < n_stream; ++i) {
                if (!__all_sync(0xffffffffu, ok)) break;
                // single buffers: T(i, 1) may overwrite T(i, 0) once the elementwise warps have read it (PREADY 0), and
                // is issued behind acc(i, 0), so that its completion also says E(i, 0) has been consumed; the next
                // tile's copy waits until acc(i, 1) has read this tile's buffer for the last time
                ok = ok && mbar_wait(BAR(B_PREADY + 0), i & 1);
                tc_fence_after_sync();
                issue_acc(i, 0);
                issue_t(i, 1);
                ok = ok && mbar_wait(BAR(B_PREADY + 1), i & 1);
                tc_fence_after_sync();
                issue_acc(i, 1);
                if (i + 1 < n_stream) {
                    ok = ok && mbar_wait(BAR(B_EMPTY), i & 1);
                    load_stream(i + 1);
                    ok = ok && mbar_wait(BAR(B_FULL), (i + 1) & 1);
                    fix_tail(i + 1);
                    tc_fence_after_sync();
                    issue_t(i + 1, 0);
                }
            }
            if (elected) mma_commit(BAR(B_DONE));
            if (!ok && lane == 0) atomicCAS(&g_bwd_error, 0, ERR_BWD);
        }
        __syncwarp();
    } else {
        // =========================== elementwise + epilogue ===============================
        // Warps w and w + 4 share TMEM lane quarter w (a warp may only touch lanes 32 (w % 4) ...) and split
        // the columns: column group cg takes the 32-column chunks 2 h + cg of each half tile.
        const int L = (warp & 3) * 32 + lane;              // TMEM lane: key (MODE_DKV) or row (MODE_DQ) own0 + L
        const int cg = warp >> 2;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;
        bool ok = true;
        // per-lane quantities
        const int own_idx = own0 + L;
        float m2_lane = 0.f, il_lane = 0.f, D_lane = 0.f;
        int pos_lane = 0;
        bool own_ok;
        if (MODE == MODE_DQ) {
            own_ok = own_idx < p.R;
            if (own_ok) {
                const size_t r = (size_t)g * p.R + own_idx;
                const float lv = p.l[r];
                m2_lane = p.m[r] * 1.4426950408889634f;
                il_lane = lv > 0.f ? 1.f / lv : 0.f;
                D_lane = p.D[r];
                pos_lane = own_idx % p.Sq;
            }
        } else {
            own_ok = own_idx < p.Skv;
        }
        for (int i = 0; i < n_stream && active; ++i) {
            const int str0 = (s_first + i) * TILE;
            float *vb = vec + (i & 1) * 4 * TILE;
            if (MODE == MODE_DKV) {
                // row statistics of the streamed rows, one per thread
                const int r = str0 + L;
                float mv = 0.f, il = 0.f, dv = 0.f;
                int last_key = -1;                  // last key this row may see (none for rows past the end)
                if (r < p.R) {
                    const size_t rr = (size_t)g * p.R + r;
                    const float lv = p.l[rr];
                    mv = p.m[rr] * 1.4426950408889634f;
                    il = lv > 0.f ? 1.f / lv : 0.f;
                    dv = p.D[rr];
                    last_key = p.causal ? (r % p.Sq) + off : p.Skv - 1;
                }
                if (cg == 0) {
                    vb[L] = mv; vb[TILE + L] = il; vb[2 * TILE + L] = dv;
                    reinterpret_cast<int *>(vb)[3 * TILE + L] = last_key;
                }
                named_bar_sync(1, 256);
            }
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {                  // half tile; this thread's chunk of it is cc
                const int cc = 2 * h + cg;
                if (ok) ok = mbar_wait(BAR(B_SREADY + h), i & 1);
                tc_fence_after_sync();
                uint32_t t1[32], t2[32];
                tmem_ld32(tmem + lane_base + C_T1 + (2 * hbuf_of(h) + cg) * 32, t1);
                tmem_ld32(tmem + lane_base + C_T2 + (2 * hbuf_of(h) + cg) * 32, t2);
                tmem_wait_ld();
                uint32_t e1[16], e2[16];
                // Is every score of this warp's 32 x 32 block visible (no key past the end, no causal mask)?  Then the
                // per-score visibility tests are skipped.  The answer is the same in every lane of the warp.
                bool all_vis;
                if (MODE == MODE_DKV) {
                    const int r_first = str0 + cc * 32, r_last = r_first + 31;
                    all_vis = r_last < p.R && own0 + TILE - 1 < p.Skv &&
                              (!p.causal || (r_first / p.Sq == r_last / p.Sq && own0 + TILE - 1 <= (r_first % p.Sq) + off));
                } else {
                    const int key_last = str0 + cc * 32 + 31;
                    all_vis = __all_sync(0xffffffffu, own_ok && key_last < p.Skv && (!p.causal || key_last <= pos_lane + off));
                }
                auto block = [&](auto fast_tag) {
                constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    // four consecutive columns (streamed indices) at a time: their row statistics come as
                    // one 16-byte shared-memory read per array (MODE_DKV) or from registers (MODE_DQ)
                    const int c0 = cc * 32 + j;
                    float m2[4], il[4], dd[4];
                    bool vis[4] = {true, true, true, true};
                    if (MODE == MODE_DKV) {
                        const float4 a = *reinterpret_cast<const float4 *>(vb + c0);
                        const float4 b = *reinterpret_cast<const float4 *>(vb + TILE + c0);
                        const float4 d = *reinterpret_cast<const float4 *>(vb + 2 * TILE + c0);
                        m2[0] = a.x; m2[1] = a.y; m2[2] = a.z; m2[3] = a.w;
                        il[0] = b.x; il[1] = b.y; il[2] = b.z; il[3] = b.w;
                        dd[0] = d.x; dd[1] = d.y; dd[2] = d.z; dd[3] = d.w;
                        if (!FAST) {
                            const int4 k = *reinterpret_cast<const int4 *>(vb + 3 * TILE + c0);
                            vis[0] = own_ok && own_idx <= k.x; vis[1] = own_ok && own_idx <= k.y;
                            vis[2] = own_ok && own_idx <= k.z; vis[3] = own_ok && own_idx <= k.w;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int key = str0 + c0 + e;
                            m2[e] = m2_lane; il[e] = il_lane; dd[e] = D_lane;
                            if (!FAST) vis[e] = own_ok && key < p.Skv && (!p.causal || key <= pos_lane + off);
                        }
                    }
                    float pv[4], dsv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float pr = (FAST || vis[e]) ? fast_exp2(fmaf(__uint_as_float(t1[j + e]), sl2, -m2[e])) * il[e] : 0.f;
                        pv[e] = pr;
                        dsv[e] = (FAST || vis[e]) ? pr * (__uint_as_float(t2[j + e]) - dd[e]) : 0.f;
                    }
#pragma unroll
                    for (int e = 0; e < 4; e += 2) {
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(pv[e], pv[e + 1]);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(dsv[e], dsv[e + 1]);
                        e1[(j + e) >> 1] = *reinterpret_cast<uint32_t *>(&h1);
                        e2[(j + e) >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                    }
                }
                };
                if (all_vis) block(std::true_type{});
                else block(std::false_type{});
                // A-operand layout of the half tile: 8x8 core matrices, K (the streamed index) inside a core row
                const int rowoff = hbuf_of(h) * E_BYTES + (L >> 3) * E_SBO + (L & 7) * 16 + (cc & 1) * 4 * 128;
#pragma unroll
                for (int kc = 0; kc < 4; ++kc) {
                    if (MODE == MODE_DKV)
                        *reinterpret_cast<uint4 *>(sE1 + rowoff + kc * 128) =
                            make_uint4(e1[4 * kc], e1[4 * kc + 1], e1[4 * kc + 2], e1[4 * kc + 3]);
                    *reinterpret_cast<uint4 *>(sE2 + rowoff + kc * 128) =
                        make_uint4(e2[4 * kc], e2[4 * kc + 1], e2[4 * kc + 2], e2[4 * kc + 3]);
                }
                tc_fence_before_sync();
                fence_proxy_async_smem();
                named_bar_sync(1, 256);
                if (L == 0 && cg == 0) mbar_arrive(BAR(B_PREADY + h));
            }
        }
        if (active) {
            if (ok) ok = mbar_wait(BAR(B_DONE), 0);
            tc_fence_after_sync();
        }
        if (!ok) atomicCAS(&g_bwd_error, 0, ERR_BWD);
        const bool have = active && ok;
        // ---- epilogue: one output row per thread -------------------------------------------
        if (MODE == MODE_DKV) {
            float *dv_row = static_cast<float *>(p.dV) + ((size_t)g * p.Skv + (own_ok ? own_idx : 0)) * D;
            float *dk_row = static_cast<float *>(p.dK) + ((size_t)g * p.Skv + (own_ok ? own_idx : 0)) * D;
            {
                const int cc = cg;
                uint32_t a[32], b[32];
                if (have) {
                    tmem_ld32(tmem + lane_base + C_ACC1 + cc * 32, a);
                    tmem_ld32(tmem + lane_base + C_ACC2 + cc * 32, b);
                    tmem_wait_ld();
                }
                if (own_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    *reinterpret_cast<float4 *>(dv_row + cc * 32 + j) =
                        have ? make_float4(__uint_as_float(a[j]), __uint_as_float(a[j + 1]), __uint_as_float(a[j + 2]), __uint_as_float(a[j + 3]))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4 *>(dk_row + cc * 32 + j) =
                        have ? make_float4(__uint_as_float(b[j]) * p.scale, __uint_as_float(b[j + 1]) * p.scale,
                                           __uint_as_float(b[j + 2]) * p.scale, __uint_as_float(b[j + 3]) * p.scale)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                }
            }
        } else {
            __nv_bfloat16 *dq_row = static_cast<__nv_bfloat16 *>(p.dQ) + ((size_t)g * p.R + (own_ok ? own_idx : 0)) * D;
            {
                const int cc = cg;
                uint32_t b[32];
                if (have) {
                    tmem_ld32(tmem + lane_base + C_ACC2 + cc * 32, b);
                    tmem_wait_ld();
                }
                if (own_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float x = have ? __uint_as_float(b[j + 2 * e]) * p.scale : 0.f;
                        const float y = have ? __uint_as_float(b[j + 2 * e + 1]) * p.scale : 0.f;
                        __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
                        w[e] = *reinterpret_cast<uint32_t *>(&h);
                    }
                    *reinterpret_cast<uint4 *>(dq_row + cc * 32 + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == CTRL_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace tcb

bool bwd_tensor_supported(const BwdProblem &p, int dtype, int grads_f32) {
    if (dtype != FDMLA_BF16 || !grads_f32) return false;
    if (p.d_qk != tcb::D || p.d_v != tcb::D || p.V == nullptr) return false;
    if (p.G <= 0 || p.R <= 0 || p.Skv <= 0 || p.Sq <= 0 || p.G > 65535) return false;
    if ((long long)p.G * p.R > 2147483647LL - 256 || (long long)p.G * p.Skv > 2147483647LL - 256) return false;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p.Q) | reinterpret_cast<uintptr_t>(p.K) | reinterpret_cast<uintptr_t>(p.V) |
                        reinterpret_cast<uintptr_t>(p.dO) | reinterpret_cast<uintptr_t>(p.dQ) | reinterpret_cast<uintptr_t>(p.dK) |
                        reinterpret_cast<uintptr_t>(p.dV);
    return (a & 15) == 0;
}

// dQ, dK (fp32), dV (fp32) from Q, K, V, dO, m, l and D = rowsum(dO o O), which the caller has computed.
int launch_bwd_tensor(const BwdProblem &p, cudaStream_t stream) {
    CUtensorMap tmQ, tmdO, tmK, tmV;
    const long long qrows = (long long)p.G * p.R, krows = (long long)p.G * p.Skv;
    if (!make_tensor_map_bf16(&tmQ, p.Q, qrows, tcb::D, tcb::TILE) || !make_tensor_map_bf16(&tmdO, p.dO, qrows, tcb::D, tcb::TILE) ||
        !make_tensor_map_bf16(&tmK, p.K, krows, tcb::D, tcb::TILE) || !make_tensor_map_bf16(&tmV, p.V, krows, tcb::D, tcb::TILE))
        return FDMLA_ERR_CUDA;
    auto kdkv = tcb::bwd_tc_kernel<tcb::MODE_DKV>;
    auto kdq = tcb::bwd_tc_kernel<tcb::MODE_DQ>;
    if (cudaFuncSetAttribute(kdkv, cudaFuncAttributeMaxDynamicSharedMemorySize, tcb::SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(kdq, cudaFuncAttributeMaxDynamicSharedMemorySize, tcb::SMEM_BYTES) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    if (tcb::LEAN &&
        (cudaFuncSetAttribute(kdkv, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
         cudaFuncSetAttribute(kdq, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess))
        return FDMLA_ERR_CUDA;
    kdkv<<<dim3((p.Skv + tcb::TILE - 1) / tcb::TILE, p.G), tcb::THREADS, tcb::SMEM_BYTES, stream>>>(p, tmQ, tmdO, tmK, tmV);
    int rc = check_launch();
    if (rc) return rc;
    kdq<<<dim3((p.R + tcb::TILE - 1) / tcb::TILE, p.G), tcb::THREADS, tcb::SMEM_BYTES, stream>>>(p, tmQ, tmdO, tmK, tmV);
    return check_launch();
}

int bwd_tensor_error_flag(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tcb::g_bwd_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int z = 0;
        cudaMemcpyToSymbol(tcb::g_bwd_error, &z, sizeof(int));
    }
    return v;
}

}  // namespace fdmla
