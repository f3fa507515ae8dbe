// Two-CTA tensor-core Flash-DMLA forward for the MLA head dimensions
// (d_qk = 576, d_v = 512, bf16) on sm_100a.
//
// A 128-row tile (the 128 heads of a decode step, or 128 consecutive queries of
// a prefill) is owned by a CLUSTER of two CTAs running tcgen05.mma with
// cta_group::2, M = 128: each CTA holds 64 of the rows.  That is what makes the
// 512-wide output fit: 64 rows x 512 fp32 columns occupy 128 TMEM lanes x 256
// columns per CTA, leaving room for a double-buffered S, and each CTA keeps only
// its 64 rows of Q (72 KB) in shared memory, leaving room for a KV ring.
//
// Per 64-key tile and per CTA (rank r of the pair):
//   S = Q K^T   A: own 64 rows of Q        B: own 32 keys x 576 (K-major)
//               D: 64 rows x 64 keys -> TMEM lanes 0-63 hold keys 0-31,
//                  lanes 64-127 hold keys 32-63
//   O += P V    A: own 64 rows of P        B: all 64 keys x own 256 columns of
//               d_v (MN-major), as two N = 256 MMAs whose halves come from the
//               two CTAs; D: lanes 0-63 hold d_v [0,256), lanes 64-127 [256,512)
// so each CTA loads (32 x 576 + 64 x 256) elements per tile with TMA (no
// multicast anywhere).  Only the leader CTA (rank 0) issues MMAs; completion is
// broadcast to both CTAs' mbarriers with tcgen05.commit.  CTA 1 forwards "my
// loads have landed" and "my P is written" to the leader with remote mbarrier
// arrivals.
//
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (leader) / load relay
// (peer) and TMEM owner, warps 2-5 softmax (thread L owns TMEM lane L: row
// L % 64, key half L / 64 of every tile) and epilogue.
//
// The recurrence is the online softmax of the reference's
// csrc/attention/fa2_fwd.cu:88-128 in base 2; O stays un-normalised until the
// epilogue and is rescaled only when the running maximum grows by more than 2^8.
// (Included by tc_fwd.cu: both kernels share the device-side error flag, which has to
// live in one translation unit.)
#pragma once

namespace fdmla {

namespace tc2 {

constexpr int T = 64;                 // keys per tile (pair-wide)
constexpr int STAGES = 2;
constexpr int NQC = 9;                // 64-column chunks of d_qk
constexpr int Q_CHUNK = 64 * 128;     // 64 rows x 128 B
constexpr int Q_BYTES = NQC * Q_CHUNK;            // 73 728
constexpr int KA_CHUNK = 32 * 128;    // own 32 keys x 128 B
constexpr int KA_BYTES = NQC * KA_CHUNK;          // 36 864
constexpr int VB_CHUNK = 64 * 128;    // 64 keys x 128 B
constexpr int VB_BYTES = 4 * VB_CHUNK;            // 32 768
constexpr int STAGE_BYTES = KA_BYTES + VB_BYTES;  // 69 632
constexpr int P_BYTES = 64 * T * 2;               // 8 192
constexpr int P_SBO = (T / 8) * 128;              // 1 024
constexpr int RED_BYTES = 2 * 128 * 4;
constexpr int O_COLS = 256, S_COL0 = 256, S_COLS = 32, TMEM_COLS = 512;
// barriers
constexpr int B_QFULL = 0, B_PEER_QFULL = 1, B_KVFULL = 2, B_PEER_FULL = B_KVFULL + STAGES,
              B_KVEMPTY = B_PEER_FULL + STAGES, B_KVFIX = B_KVEMPTY + STAGES, B_SFULL = B_KVFIX + 1,
              B_PFULL = B_SFULL + 2, B_OREADY = B_PFULL + 1, NBARS = B_OREADY + 1;
constexpr int SMEM_BYTES = 1024 + Q_BYTES + STAGES * STAGE_BYTES + P_BYTES + RED_BYTES + NBARS * 8 + 16;
static_assert(SMEM_BYTES <= kMaxSmemPerBlock, "shared memory overflow");
constexpr int THREADS = 192;
enum { ERR_PRODUCER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_PAGE = 4, ERR_RELAY = 14 };

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
fwd_tc2_kernel(const FwdProblem p, const __grid_constant__ CUtensorMap tmQ,
               const __grid_constant__ CUtensorMap tmK32, const __grid_constant__ CUtensorMap tmK64) {
    using namespace ptx;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sQ = smem;
    uint8_t *sKV = sQ + Q_BYTES;
    uint8_t *sP = sKV + STAGES * STAGE_BYTES;
    float *red = reinterpret_cast<float *>(sP + P_BYTES);       // [2][128]
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(red) + RED_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;

    // ---- work item (identical in both CTAs of the pair) ---------------------------
    const int n_row_tiles = (p.R + 127) / 128;
    int tile_idx = blockIdx.x >> 1;
    if (p.causal) tile_idx = n_row_tiles - 1 - tile_idx;
    const int g = blockIdx.y, split = blockIdx.z;
    const int row0 = tile_idx * 128;
    const int seq = p.seqlens ? p.seqlens[g] : p.Skv;
    const int w_lo = p.kv_begin > 0 ? p.kv_begin : 0;
    const int w_hi = (p.kv_end >= 0 && p.kv_end < seq) ? p.kv_end : seq;
    int lo, hi;
    split_window(w_lo, w_hi, p.page_table ? p.page_size : T, split, p.num_splits, &lo, &hi);
    const int rows_here = (p.R - row0) < 128 ? (p.R - row0) : 128;
    int blk_vis = seq;
    if (p.causal) {
        const int r_last = row0 + rows_here - 1;
        const int i_max = (row0 / p.Sq == r_last / p.Sq) ? (r_last % p.Sq) : (p.Sq - 1);
        long long v = (long long)i_max + seq - p.Sq + 1;
        blk_vis = v < 0 ? 0 : (v > seq ? seq : (int)v);
    }
    const int blk_hi = hi < blk_vis ? hi : blk_vis;
    const int t_begin = (lo / T) * T;
    const int err_now = *reinterpret_cast<volatile int *>(&g_tc_error);
    const bool poisoned = err_now != 0 && err_now != ERR_PAGE;
    const int n_tiles = (blk_hi > lo && !poisoned) ? (blk_hi - t_begin + T - 1) / T : 0;

    // ---- set-up ------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        mbar_init(BAR(B_QFULL), 1);
        mbar_init(BAR(B_PEER_QFULL), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(BAR(B_KVFULL + s), 1);
            mbar_init(BAR(B_PEER_FULL + s), 1);
            mbar_init(BAR(B_KVEMPTY + s), 1);
        }
        mbar_init(BAR(B_KVFIX), 1);
        mbar_init(BAR(B_SFULL + 0), 1);
        mbar_init(BAR(B_SFULL + 1), 1);
        mbar_init(BAR(B_PFULL), 2);          // one arrival per CTA of the pair
        mbar_init(BAR(B_OREADY), 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_2cta(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish_2cta();
    }
    tc_fence_before_sync();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();                      // the peer's barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // =========================== TMA producer (both CTAs) ============================
        if (n_tiles > 0) {
            if (lane == 0) {
                prefetch_tmap(&tmQ);
                prefetch_tmap(&tmK32);
                prefetch_tmap(&tmK64);
                mbar_arrive_expect_tx(BAR(B_QFULL), Q_BYTES);
                const int qrow = g * p.R + row0 + 64 * (int)rank;
                for (int c = 0; c < NQC; ++c)
                    tma_load_2d(smem_u32(sQ + c * Q_CHUNK), &tmQ, c * 64, qrow, BAR(B_QFULL));
            }
            bool ok = true;
            for (int t = 0; t < n_tiles; ++t) {
                const int stage = t % STAGES;
                if (t >= STAGES) ok = mbar_wait(BAR(B_KVEMPTY + stage), ((t / STAGES) - 1) & 1);
                if (!ok) { if (lane == 0) atomicCAS(&g_tc_error, 0, ERR_PRODUCER); break; }
                const int t0 = t_begin + t * T;
                uint8_t *st = sKV + stage * STAGE_BYTES;
                if (lane == 0) {
                    long long row;
                    if (p.page_table) {
                        const int lp = t0 / p.page_size;
                        int pg = lp < p.max_pages ? p.page_table[(size_t)g * p.max_pages + lp] : -1;
                        if (pg < 0 || pg >= p.num_pages) { atomicCAS(&g_tc_error, 0, ERR_PAGE); pg = 0; }
                        row = (long long)pg * p.page_size + (t0 - lp * p.page_size);
                    } else {
                        row = (long long)g * p.Skv + t0;
                    }
                    mbar_arrive_expect_tx(BAR(B_KVFULL + stage), STAGE_BYTES);
                    // own 32 keys, all 576 columns (B operand of Q K^T)
                    for (int c = 0; c < NQC; ++c)
                        tma_load_2d(smem_u32(st + c * KA_CHUNK), &tmK32, c * 64, (int)row + 32 * (int)rank,
                                    BAR(B_KVFULL + stage));
                    // all 64 keys, own 256 columns of d_v (B operand of P V)
                    for (int c = 0; c < 4; ++c)
                        tma_load_2d(smem_u32(st + KA_BYTES + c * VB_CHUNK), &tmK64, 256 * (int)rank + c * 64, (int)row,
                                    BAR(B_KVFULL + stage));
                }
                if (t0 + T > seq) {
                    // keys past the end of the sequence: zero their V rows once the copy has landed
                    ok = mbar_wait(BAR(B_KVFULL + stage), (t / STAGES) & 1);
                    if (!ok) { if (lane == 0) atomicCAS(&g_tc_error, 0, ERR_PRODUCER); break; }
                    const int first_bad = seq > t0 ? seq - t0 : 0;
                    const int bad_rows = T - first_bad;
                    for (int idx = lane; idx < 4 * bad_rows * 8; idx += 32) {
                        const int ch = idx / (bad_rows * 8), rem = idx - ch * bad_rows * 8;
                        const int r = first_bad + rem / 8, q16 = rem & 7;
                        *reinterpret_cast<uint4 *>(st + KA_BYTES + ch * VB_CHUNK + r * 128 + q16 * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(B_KVFIX));
                }
            }
        }
    } else if (warp == 1) {
        if (leader) {
            // =========================== MMA issuer (leader CTA) =========================
            if (lane == 0 && n_tiles > 0) {
                constexpr uint32_t idesc_qk = make_idesc_bf16(128, T, 0, 0);
                constexpr uint32_t idesc_pv = make_idesc_bf16(128, 256, 0, 1);
                const uint32_t sQ_a = smem_u32(sQ), sKV_a = smem_u32(sKV), sP_a = smem_u32(sP);
                bool ok = mbar_wait(BAR(B_QFULL), 0) && mbar_wait_cluster(BAR(B_PEER_QFULL), 0);
                auto issue_qk = [&](int t) -> bool {
                    const int stage = t % STAGES, b = t & 1;
                    if (!mbar_wait(BAR(B_KVFULL + stage), (t / STAGES) & 1)) return false;
                    if (t_begin + t * T + T > seq && !mbar_wait(BAR(B_KVFIX), 0)) return false;
                    if (!mbar_wait_cluster(BAR(B_PEER_FULL + stage), (t / STAGES) & 1)) return false;
                    tc_fence_after_sync();
                    const uint32_t kbase = sKV_a + stage * STAGE_BYTES;
#pragma unroll
                    for (int c = 0; c < NQC; ++c) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t da = make_smem_desc(sQ_a + c * Q_CHUNK + k * 32, 16, 1024, kLayoutSw128);
                            const uint64_t db = make_smem_desc(kbase + c * KA_CHUNK + k * 32, 16, 1024, kLayoutSw128);
                            mma_bf16_ss_2cta(tmem + S_COL0 + b * S_COLS, da, db, idesc_qk, (c | k) != 0);
                        }
                    }
                    mma_commit_2cta(BAR(B_SFULL + b), 3);
                    return true;
                };
                if (ok) ok = issue_qk(0);
                for (int t = 0; t < n_tiles && ok; ++t) {
                    if (t + 1 < n_tiles) ok = issue_qk(t + 1);
                    if (!ok) break;
                    ok = mbar_wait_cluster(BAR(B_PFULL), t & 1);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const int stage = t % STAGES;
                    const uint32_t vbase = sKV_a + stage * STAGE_BYTES + KA_BYTES;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
#pragma unroll
                        for (int ks = 0; ks < T / 16; ++ks) {
                            const uint64_t da = make_smem_desc(sP_a + ks * 256, 128, P_SBO, kLayoutNone);
                            const uint64_t db = make_smem_desc(vbase + j * 2 * VB_CHUNK + ks * 2048, VB_CHUNK, 1024, kLayoutSw128);
                            mma_bf16_ss_2cta(tmem + j * 128, da, db, idesc_pv, (t | ks) != 0);
                        }
                    }
                    mma_commit_2cta(BAR(B_KVEMPTY + stage), 3);
                    mma_commit_2cta(BAR(B_OREADY), 3);
                }
                if (!ok) atomicCAS(&g_tc_error, 0, ERR_MMA);
            }
        } else {
            // =========================== load relay (peer CTA) ===========================
            if (lane == 0 && n_tiles > 0) {
                bool ok = mbar_wait(BAR(B_QFULL), 0);
                if (ok) mbar_arrive_cluster(map_to_cta(BAR(B_PEER_QFULL), 0));
                for (int t = 0; t < n_tiles && ok; ++t) {
                    const int stage = t % STAGES;
                    ok = mbar_wait(BAR(B_KVFULL + stage), (t / STAGES) & 1);
                    if (ok && t_begin + t * T + T > seq) ok = mbar_wait(BAR(B_KVFIX), 0);
                    if (ok) mbar_arrive_cluster(map_to_cta(BAR(B_PEER_FULL + stage), 0));
                }
                if (!ok) atomicCAS(&g_tc_error, 0, ERR_RELAY);
            }
        }
        __syncwarp();
    } else {
        // =========================== softmax + epilogue (both CTAs) ========================
        const int L = (warp & 3) * 32 + lane;          // TMEM lane owned by this thread
        const int row = L & 63, half = L >> 6;
        const int rr = row0 + 64 * (int)rank + row;
        const bool row_ok = rr < p.R;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        int upper = lo;
        if (row_ok) {
            long long vis = seq;
            if (p.causal) {
                vis = (long long)(rr % p.Sq) + seq - p.Sq + 1;
                vis = vis < 0 ? 0 : (vis > seq ? seq : vis);
            }
            upper = (int)(vis < hi ? vis : hi);
            if (upper < lo) upper = lo;
        }
        const float sl2 = p.scale * 1.4426950408889634f;
        float m_true = -CUDART_INF_F, m_ref = -CUDART_INF_F, l_run = 0.f;   // l_run: this thread's key half only
        const uint32_t pfull_leader = map_to_cta(BAR(B_PFULL), 0);
        bool ok = true;
        uint32_t r[32];
        for (int t = 0; t < n_tiles; ++t) {
            const int b = t & 1, tok0 = t_begin + t * T + 32 * half;
            // after a failed wait the loop keeps running without further waits so that the
            // named barriers below stay matched across the 128 softmax threads
            if (ok) ok = mbar_wait(BAR(B_SFULL + b), (t / 2) & 1);
            tc_fence_after_sync();
            tmem_ld32(tmem + lane_base + S_COL0 + b * S_COLS, r);
            tmem_wait_ld();
            float tmax = -CUDART_INF_F;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int tok = tok0 + j;
                const float v = (tok >= lo && tok < upper) ? __uint_as_float(r[j]) * sl2 : -CUDART_INF_F;
                r[j] = __float_as_uint(v);
                tmax = fmaxf(tmax, v);
            }
            // the row's other key half lives in the thread 64 lanes away
            red[(t & 1) * 128 + L] = tmax;
            named_bar_sync(1, 128);
            tmax = fmaxf(tmax, red[(t & 1) * 128 + (L ^ 64)]);
            const float m_new = fmaxf(m_true, tmax);
            const bool need = m_new > m_ref + 8.f;
            if (t > 0) {
                if (ok) ok = mbar_wait(BAR(B_OREADY), (t - 1) & 1);
                tc_fence_after_sync();
            }
            if (__any_sync(0xffffffffu, need)) {
                float alpha = 1.f;
                if (need) {
                    alpha = (m_ref == -CUDART_INF_F) ? 0.f : fast_exp2(m_ref - m_new);
                    l_run *= alpha;
                    m_ref = m_new;
                }
                if (t > 0) {
                    uint32_t o[32];
#pragma unroll 1
                    for (int cc = 0; cc < O_COLS / 32; ++cc) {
                        tmem_ld32(tmem + lane_base + cc * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                        tmem_st32(tmem + lane_base + cc * 32, o);
                    }
                    tmem_wait_st();
                }
            }
            m_true = m_new;
            float lsum = 0.f;
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
                const float p0 = (v0 == -CUDART_INF_F) ? 0.f : fast_exp2(v0 - m_ref);
                const float p1 = (v1 == -CUDART_INF_F) ? 0.f : fast_exp2(v1 - m_ref);
                lsum += p0 + p1;
                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h);
            }
            l_run += lsum;
            uint8_t *prow = sP + (row >> 3) * P_SBO + (row & 7) * 16 + half * 4 * 128;
#pragma unroll
            for (int kc = 0; kc < 4; ++kc)
                *reinterpret_cast<uint4 *>(prow + kc * 128) =
                    make_uint4(packed[4 * kc], packed[4 * kc + 1], packed[4 * kc + 2], packed[4 * kc + 3]);
            tc_fence_before_sync();
            fence_proxy_async_smem();
            named_bar_sync(2, 128);
            if (L == 0) mbar_arrive_cluster(pfull_leader);
        }
        if (ok && n_tiles > 0) {
            ok = mbar_wait(BAR(B_OREADY), (n_tiles - 1) & 1);
            tc_fence_after_sync();
        }
        if (!ok) atomicCAS(&g_tc_error, 0, ERR_SOFTMAX);
        // row sum = both key halves
        named_bar_sync(1, 128);
        red[L] = l_run;
        named_bar_sync(2, 128);
        const float l_tot = l_run + red[L ^ 64];
        // ---- epilogue: thread L writes row `row`, d_v columns [256*half, 256*half + 256) ----
        const bool have = ok && n_tiles > 0 && l_tot > 0.f;
        const float inv = have ? 1.f / l_tot : 0.f;
        const bool final_out = (p.num_splits == 1 && p.O != nullptr);
        const size_t grow = (size_t)g * p.R + (row_ok ? rr : 0);
        const size_t prow_idx = (size_t)split * p.G * p.R + grow;
        const int col0 = 256 * half;
#pragma unroll 1
        for (int cc = 0; cc < O_COLS / 32; ++cc) {
            uint32_t o[32];
            if (n_tiles > 0 && ok) {
                tmem_ld32(tmem + lane_base + cc * 32, o);
                tmem_wait_ld();
            }
            if (!row_ok) continue;
            if (final_out) {
                __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.O) + grow * p.d_v + col0 + cc * 32;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = have ? __uint_as_float(o[j + 2 * e]) * inv : 0.f;
                        const float c = have ? __uint_as_float(o[j + 2 * e + 1]) * inv : 0.f;
                        __nv_bfloat162 h = __floats2bfloat162_rn(a, c);
                        w[e] = *reinterpret_cast<uint32_t *>(&h);
                    }
                    *reinterpret_cast<uint4 *>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
                float *dst = p.O_part + prow_idx * p.d_v + col0 + cc * 32;
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(dst + j) =
                        make_float4(have ? __uint_as_float(o[j]) * inv : 0.f, have ? __uint_as_float(o[j + 1]) * inv : 0.f,
                                    have ? __uint_as_float(o[j + 2]) * inv : 0.f, have ? __uint_as_float(o[j + 3]) * inv : 0.f);
            }
        }
        if (row_ok && half == 0) {
            const float m_out = have ? m_true * 0.6931471805599453f : -CUDART_INF_F;
            const float l_out = have ? l_tot * fast_exp2(m_ref - m_true) : 0.f;
            if (final_out) { p.m[grow] = m_out; p.l[grow] = l_out; }
            else { p.m_part[prow_idx] = m_out; p.l_part[prow_idx] = l_out; }
        }
    }

    // ---- teardown: neither CTA may leave while the pair can still touch its memory --------
    tc_fence_before_sync();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_2cta(tmem, TMEM_COLS);
    }
}

}  // namespace tc2

// --------------------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------------------
bool fwd_tensor2_supported(const FwdProblem &p, int dtype) {
    if (dtype != FDMLA_BF16) return false;
    if (p.d_qk != 576 || p.d_v != 512 || p.V != nullptr) return false;
    if (p.page_table && (p.page_size % tc2::T) != 0) return false;
    if (p.G <= 0 || p.R <= 0 || p.G > 65535 || p.num_splits > 65535) return false;
    const long long kv_rows = p.page_table ? (long long)p.num_pages * p.page_size : (long long)p.G * p.Skv;
    if (kv_rows <= 0 || kv_rows > 2147483647LL || (long long)p.G * p.R > 2147483647LL) return false;
    if ((reinterpret_cast<uintptr_t>(p.Q) | reinterpret_cast<uintptr_t>(p.K)) & 15) return false;
    if ((reinterpret_cast<uintptr_t>(p.O) | reinterpret_cast<uintptr_t>(p.O_part)) & 15) return false;
    return true;
}

int launch_fwd_tensor2(const FwdProblem &p, cudaStream_t stream) {
    CUtensorMap tmQ, tmK32, tmK64;
    const long long kv_rows = p.page_table ? (long long)p.num_pages * p.page_size : (long long)p.G * p.Skv;
    if (!make_tensor_map_bf16(&tmQ, p.Q, (long long)p.G * p.R, p.d_qk, 64)) return FDMLA_ERR_CUDA;
    if (!make_tensor_map_bf16(&tmK32, p.K, kv_rows, p.d_qk, 32)) return FDMLA_ERR_CUDA;
    if (!make_tensor_map_bf16(&tmK64, p.K, kv_rows, p.d_qk, 64)) return FDMLA_ERR_CUDA;
    if (cudaFuncSetAttribute(tc2::fwd_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2::SMEM_BYTES) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    dim3 grid(((p.R + 127) / 128) * 2, p.G, p.num_splits);
    tc2::fwd_tc2_kernel<<<grid, tc2::THREADS, tc2::SMEM_BYTES, stream>>>(p, tmQ, tmK32, tmK64);
    return check_launch();
}

}  // namespace fdmla
