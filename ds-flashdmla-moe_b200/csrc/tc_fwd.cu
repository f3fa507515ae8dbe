// Tensor-core Flash-DMLA forward for sm_100a: tcgen05.mma with the S and O
// accumulators in tensor memory, operands staged in shared memory by TMA
// (128-byte swizzle, never multicast), warp-specialised roles:
//   warp 0      TMA producer (Q once, then the KV tile ring; zero-fills rows
//               past the end of a sequence so stale cache contents never
//               reach the P*V product)
//   warp 1      MMA issuer (one elected thread) and TMEM owner
//   warps 2-5   online softmax, one thread per query row (tcgen05.ld of S,
//               lazy rescale of O in TMEM, P written to shared memory as the
//               A operand of P*V), then the epilogue
// One CTA owns 128 query rows of one KV group (128 heads of a decode step, or
// 128 consecutive queries of a prefill) and one slice of d_v, for one split of
// the key range.  The latent tile loaded once serves as the K-major B operand
// of Q*K^T and, its first d_v columns, as the MN-major B operand of P*V.
//
// The recurrence is the online softmax of the reference's
// csrc/attention/fa2_fwd.cu:88-128 in base 2, with O left un-normalised until
// the epilogue and rescaled only when the running maximum grows by more than
// 2^8 (the row statistics written out are exact: m is the true maximum).
#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace fdmla {

__device__ int g_tc_error = 0;   // first time-out code seen by any CTA (0 = none)

template <int NQC_, int NVC_, int T_, int STAGES_, bool SEPV_, int VSPLIT_, int NSBUF_ = 2, int CTAS_PER_SM_ = 1>
struct TcCfg {
    static constexpr int NSBUF = NSBUF_;    // S accumulators in tensor memory (2: Q K^T of the next tile runs under the softmax)
    static constexpr int CTAS_PER_SM = CTAS_PER_SM_;   // CTAs meant to share an SM (launch bound; shared and tensor memory must fit)
    static constexpr int NQC = NQC_;        // 64-column chunks of d_qk
    static constexpr int NVC = NVC_;        // 64-column chunks of d_v owned by one CTA
    static constexpr int T = T_;            // keys per tile
    static constexpr int STAGES = STAGES_;  // KV ring depth
    static constexpr bool SEPV = SEPV_;     // V is its own tensor (on-the-fly latents)
    static constexpr int VSPLIT = VSPLIT_;  // CTAs sharing a row tile, each with NVC chunks of d_v
    static constexpr int M = 128;
    static constexpr int Q_CHUNK = M * 128;
    static constexpr int Q_BYTES = NQC * Q_CHUNK;
    static constexpr int KV_CHUNK = T * 128;
    static constexpr int K_BYTES = NQC * KV_CHUNK;
    static constexpr int V_BYTES = SEPV ? NVC * KV_CHUNK : 0;
    static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
    static constexpr int P_BYTES = M * T * 2;
    static constexpr int P_SBO = (T / 8) * 128;   // 8-row group stride of the un-swizzled P tile
    static constexpr int O_COLS = NVC * 64;
    static constexpr int S_COL0 = O_COLS;
    static constexpr int TMEM_COLS = (O_COLS + NSBUF * T) <= 128 ? 128 : ((O_COLS + NSBUF * T) <= 256 ? 256 : 512);
    static constexpr int NBARS = 1 + 2 * STAGES + 1 + 2 + 2 + 1 + 1;
    // room to round the dynamic shared memory up to 1 KB; two CTAs per SM only fit with 896 B of it, which is enough
    // for a base that is 128-byte aligned (the kernel checks and reports instead of running past its allocation)
    static constexpr int ALIGN_SLACK = CTAS_PER_SM > 1 ? 896 : 1024;
    static constexpr int SMEM_BYTES = ALIGN_SLACK + Q_BYTES + STAGES * STAGE_BYTES + P_BYTES + NBARS * 8 + 16;
    static constexpr int D_QK = NQC * 64;
    static constexpr int D_V = NVC * 64 * VSPLIT;
    static_assert(O_COLS + NSBUF * T <= 512 && TMEM_COLS * CTAS_PER_SM <= 512, "TMEM overflow");
    static_assert(NSBUF == 1 || NSBUF == 2, "one or two S accumulators");
    static_assert(SMEM_BYTES <= kMaxSmemPerBlock, "shared memory overflow");
    static_assert(CTAS_PER_SM * (SMEM_BYTES + 1024) <= 233472, "the CTAs meant to share an SM do not fit its 228 KB");
    static_assert(T % 32 == 0 && T <= 256, "tile size");
};

constexpr int TC_THREADS = 192;
enum TcErr { ERR_PRODUCER = 1, ERR_MMA = 2, ERR_SOFTMAX = 3, ERR_PAGE = 4 };

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <class C>
__global__ void __launch_bounds__(TC_THREADS, C::CTAS_PER_SM)
fwd_tc_kernel(const FwdProblem p, const __grid_constant__ CUtensorMap tmQ,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
    using namespace ptx;
    constexpr int T = C::T, STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sQ = smem;
    uint8_t *sKV = sQ + C::Q_BYTES;
    uint8_t *sP = sKV + STAGES * C::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sP + C::P_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::NBARS);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * i; };
    constexpr int B_QFULL = 0, B_KVFULL = 1, B_KVEMPTY = 1 + STAGES, B_KVFIX = 1 + 2 * STAGES,
                  B_SFULL = B_KVFIX + 1, B_SEMPTY = B_SFULL + 2, B_PFULL = B_SEMPTY + 2, B_OREADY = B_PFULL + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- which work item ------------------------------------------------------
    const int vsplit = blockIdx.x % C::VSPLIT;
    const int n_row_tiles = (p.R + 127) / 128;
    int tile_idx = blockIdx.x / C::VSPLIT;
    if (p.causal) tile_idx = n_row_tiles - 1 - tile_idx;   // longest key ranges first
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
    // once any CTA has reported a failed wait the rest of the grid does no work
    bool poisoned = *reinterpret_cast<volatile int *>(&g_tc_error) != 0 &&
                    *reinterpret_cast<volatile int *>(&g_tc_error) != ERR_PAGE;
    if (smem + (C::SMEM_BYTES - C::ALIGN_SLACK) > smem_raw + C::SMEM_BYTES) {     // base less aligned than assumed
        if (threadIdx.x == 0) atomicCAS(&g_tc_error, 0, ERR_PRODUCER);
        poisoned = true;
    }
    const int n_tiles = (blk_hi > lo && !poisoned) ? (blk_hi - t_begin + T - 1) / T : 0;

    // ---- set-up -----------------------------------------------------------------
    if (threadIdx.x == 0) {
        mbar_init(BAR(B_QFULL), 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(BAR(B_KVFULL + s), 1); mbar_init(BAR(B_KVEMPTY + s), 1); }
        mbar_init(BAR(B_KVFIX), 1);
        for (int b = 0; b < 2; ++b) { mbar_init(BAR(B_SFULL + b), 1); mbar_init(BAR(B_SEMPTY + b), 128); }
        mbar_init(BAR(B_PFULL), 128);
        mbar_init(BAR(B_OREADY), 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // =========================== TMA producer ===================================
        if (n_tiles > 0) {
            if (lane == 0) {
                prefetch_tmap(&tmQ);
                prefetch_tmap(&tmK);
                if (C::SEPV) prefetch_tmap(&tmV);
                mbar_arrive_expect_tx(BAR(B_QFULL), C::Q_BYTES);
                const int qrow = g * p.R + row0;
                for (int c = 0; c < C::NQC; ++c)
                    tma_load_2d(smem_u32(sQ + c * C::Q_CHUNK), &tmQ, c * 64, qrow, BAR(B_QFULL));
            }
            bool ok = true;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int stage = t % STAGES;
                if (t >= STAGES) ok = mbar_wait(BAR(B_KVEMPTY + stage), ((t / STAGES) - 1) & 1);
                if (!ok) { if (lane == 0) atomicCAS(&g_tc_error, 0, ERR_PRODUCER); break; }
                const int t0 = t_begin + t * T;
                uint8_t *st = sKV + stage * C::STAGE_BYTES;
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
                    mbar_arrive_expect_tx(BAR(B_KVFULL + stage), C::STAGE_BYTES);
                    for (int c = 0; c < C::NQC; ++c)
                        tma_load_2d(smem_u32(st + c * C::KV_CHUNK), &tmK, c * 64, (int)row, BAR(B_KVFULL + stage));
                    if (C::SEPV)
                        for (int c = 0; c < C::NVC; ++c)
                            tma_load_2d(smem_u32(st + C::K_BYTES + c * C::KV_CHUNK), &tmV, c * 64, (int)row,
                                        BAR(B_KVFULL + stage));
                }
                if (t0 + T > seq) {
                    // keys past the end of the sequence: zero their rows (whole 128-byte
                    // rows, so the swizzle does not matter) once the copy has landed
                    ok = mbar_wait(BAR(B_KVFULL + stage), (t / STAGES) & 1);
                    if (!ok) { if (lane == 0) atomicCAS(&g_tc_error, 0, ERR_PRODUCER); break; }
                    const int first_bad = seq > t0 ? seq - t0 : 0;
                    const int bad_rows = T - first_bad;
                    constexpr int NCH = C::NQC + (C::SEPV ? C::NVC : 0);
                    for (int idx = lane; idx < NCH * bad_rows * 8; idx += 32) {
                        const int ch = idx / (bad_rows * 8), rem = idx - ch * bad_rows * 8;
                        const int r = first_bad + rem / 8, q16 = rem & 7;
                        *reinterpret_cast<uint4 *>(st + ch * C::KV_CHUNK + r * 128 + q16 * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(B_KVFIX));
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer =====================================
        // The whole warp runs the loop converged and one elected lane issues (descriptor arithmetic on the
        // uniform datapath: about twice the issue rate of a lone lane of a diverged warp).
        if (n_tiles > 0) {
            const bool elected = elect_one();
            constexpr uint32_t idesc_qk = make_idesc_bf16(128, T, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_bf16(128, C::O_COLS, 0, 1);
            const uint32_t sQ_a = smem_u32(sQ), sKV_a = smem_u32(sKV), sP_a = smem_u32(sP);
            bool ok = mbar_wait(BAR(B_QFULL), 0);
            auto issue_qk = [&](int t) -> bool {
                const int stage = t % STAGES, b = t % C::NSBUF;
                if (!mbar_wait(BAR(B_KVFULL + stage), (t / STAGES) & 1)) return false;
                if (t_begin + t * T + T > seq && !mbar_wait(BAR(B_KVFIX), 0)) return false;
                if (t >= C::NSBUF && !mbar_wait(BAR(B_SEMPTY + b), ((t / C::NSBUF) - 1) & 1)) return false;
                tc_fence_after_sync();
                const uint32_t kbase = sKV_a + stage * C::STAGE_BYTES;
                if (elected) {
#pragma unroll
                    for (int c = 0; c < C::NQC; ++c) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t da = make_smem_desc(sQ_a + c * C::Q_CHUNK + k * 32, 16, 1024, kLayoutSw128);
                            const uint64_t db = make_smem_desc(kbase + c * C::KV_CHUNK + k * 32, 16, 1024, kLayoutSw128);
                            mma_bf16_ss(tmem + C::S_COL0 + b * T, da, db, idesc_qk, (c | k) != 0);
                        }
                    }
                    mma_commit(BAR(B_SFULL + b));
                }
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int t = 0; t < n_tiles; ++t) {
                if (!__all_sync(0xffffffffu, ok)) break;
                if (t + 1 < n_tiles) ok = issue_qk(t + 1);
                if (!__all_sync(0xffffffffu, ok)) break;
                ok = mbar_wait(BAR(B_PFULL), t & 1);
                if (!__all_sync(0xffffffffu, ok)) break;
                tc_fence_after_sync();
                const int stage = t % STAGES;
                const uint32_t vbase = sKV_a + stage * C::STAGE_BYTES +
                                       (C::SEPV ? C::K_BYTES : vsplit * C::NVC * C::KV_CHUNK);
                if (elected) {
#pragma unroll
                    for (int ks = 0; ks < T / 16; ++ks) {
                        const uint64_t da = make_smem_desc(sP_a + ks * 256, 128, C::P_SBO, kLayoutNone);
                        const uint64_t db = make_smem_desc(vbase + ks * 2048, C::KV_CHUNK, 1024, kLayoutSw128);
                        mma_bf16_ss(tmem, da, db, idesc_pv, (t | ks) != 0);
                    }
                    mma_commit(BAR(B_KVEMPTY + stage));
                    mma_commit(BAR(B_OREADY));
                }
            }
            if (!ok && lane == 0) atomicCAS(&g_tc_error, 0, ERR_MMA);
        }
        __syncwarp();
    } else {
        // =========================== softmax + epilogue ===============================
        const int q = warp & 3;                        // TMEM lane quarter this warp may access
        const int row_in_tile = q * 32 + lane;
        const int rr = row0 + row_in_tile;
        const bool row_ok = rr < p.R;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
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
        float m_true = -CUDART_INF_F, m_ref = -CUDART_INF_F, l_run = 0.f;
        bool ok = true;
        uint32_t r[32];
        for (int t = 0; t < n_tiles; ++t) {
            const int b = t % C::NSBUF, t0 = t_begin + t * T;
            ok = mbar_wait(BAR(B_SFULL + b), (t / C::NSBUF) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t s_addr = tmem + lane_base + C::S_COL0 + b * T;
            // pass 1: tile maximum of the visible scores (base-2 units); no per-key masking when this row sees the whole tile
            const bool all_visible = t0 >= lo && t0 + T <= upper && sl2 > 0.f;
            float tmax = -CUDART_INF_F;
            auto max_of = [&](const uint32_t (&v)[32], int cc) {
                if (all_visible) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) tmax = fmaxf(tmax, __uint_as_float(v[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int tok = t0 + cc * 32 + j;
                        if (tok >= lo && tok < upper) tmax = fmaxf(tmax, __uint_as_float(v[j]) * sl2);
                    }
                }
            };
#pragma unroll 1
            for (int cc = 0; cc < T / 32; ++cc) {
                tmem_ld32(s_addr + cc * 32, r);
                tmem_wait_ld();
                max_of(r, cc);
            }
            if (all_visible) tmax *= sl2;     // the fast path took the maximum of the raw scores (sl2 > 0)
            const float m_new = fmaxf(m_true, tmax);
            const bool need = m_new > m_ref + 8.f;       // also true for the first finite maximum
            // P*V of the previous tile must be done before O is rescaled or P overwritten
            if (t > 0) {
                ok = mbar_wait(BAR(B_OREADY), (t - 1) & 1);
                if (!ok) break;
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
                    for (int cc = 0; cc < C::O_COLS / 32; ++cc) {
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
            // pass 2: P = 2^(s - m_ref) in bf16, K-major un-swizzled core matrices
            float lsum = 0.f;
            uint8_t *prow = sP + (row_in_tile >> 3) * C::P_SBO + (row_in_tile & 7) * 16;
            auto emit_p = [&](const uint32_t (&v)[32], int cc) {
                uint32_t packed[16];
                if (all_visible) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(v[j]), sl2, -m_ref));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(v[j + 1]), sl2, -m_ref));
                        lsum += p0 + p1;
                        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const int tok = t0 + cc * 32 + j;
                        const float p0 = (tok >= lo && tok < upper) ? fast_exp2(fmaf(__uint_as_float(v[j]), sl2, -m_ref)) : 0.f;
                        const float p1 = (tok + 1 >= lo && tok + 1 < upper) ? fast_exp2(fmaf(__uint_as_float(v[j + 1]), sl2, -m_ref)) : 0.f;
                        lsum += p0 + p1;
                        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h);
                    }
                }
#pragma unroll
                for (int kc = 0; kc < 4; ++kc)
                    *reinterpret_cast<uint4 *>(prow + (cc * 4 + kc) * 128) =
                        make_uint4(packed[4 * kc], packed[4 * kc + 1], packed[4 * kc + 2], packed[4 * kc + 3]);
            };
#pragma unroll 1
            for (int cc = 0; cc < T / 32; ++cc) {
                if (T > 32) {
                    tmem_ld32(s_addr + cc * 32, r);
                    tmem_wait_ld();
                }
                emit_p(r, cc);
            }
            l_run += lsum;
            tc_fence_before_sync();
            mbar_arrive(BAR(B_SEMPTY + b));      // S[b] fully read
            fence_proxy_async_smem();            // P visible to the tensor core
            mbar_arrive(BAR(B_PFULL));
        }
        if (ok && n_tiles > 0) {
            ok = mbar_wait(BAR(B_OREADY), (n_tiles - 1) & 1);
            tc_fence_after_sync();
        }
        if (!ok) atomicCAS(&g_tc_error, 0, ERR_SOFTMAX);
        // ---- epilogue: O / l, row statistics in natural-log units ------------------
        const bool have = ok && n_tiles > 0 && l_run > 0.f;
        const float inv = have ? 1.f / l_run : 0.f;
        const bool final_out = (p.num_splits == 1 && p.O != nullptr);
        const size_t grow = (size_t)g * p.R + (row_ok ? rr : 0);
        const size_t prow_idx = (size_t)split * p.G * p.R + grow;
        const int col0 = vsplit * C::O_COLS;
#pragma unroll 1
        for (int cc = 0; cc < C::O_COLS / 32; ++cc) {
            uint32_t o[32];
            if (n_tiles > 0 && ok) {          // warp-uniform
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
        if (row_ok && vsplit == 0) {
            const float m_out = have ? m_true * 0.6931471805599453f : -CUDART_INF_F;
            const float l_out = have ? l_run * exp2f(m_ref - m_true) : 0.f;
            if (final_out) { p.m[grow] = m_out; p.l[grow] = l_out; }
            else { p.m_part[prow_idx] = m_out; p.l_part[prow_idx] = l_out; }
        }
    }

    // ---- teardown: every role has finished with TMEM --------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
}

// --------------------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------------------
using MlaCfg = TcCfg<9, 4, 32, 2, false, 2>;    // d_qk 576, d_v 512 in two 256-column halves
// 64-wide heads: three CTAs share an SM (64-key tiles, one S accumulator, two KV stages: 65 KB of shared memory and
// 128 tensor-memory columns each), so that one CTA's softmax - the exponentials bound this shape, not the MMAs - runs
// under the others' MMAs and every scheduler has three softmax warps to switch between.  Measured on config 4b's
// shape (forward with the projections): one CTA per SM with 128-key tiles and two S accumulators 1.33 ms, two CTAs
// per SM 1.00 ms, with the unmasked fast path of the softmax 0.76 ms, three CTAs with 64-key tiles 0.68 ms; keeping
// the 64 scores of a thread in registers between the two passes spills under the three-CTA register bound (0.84 ms).
using OtfCfg = TcCfg<1, 1, 64, 2, true, 1, 1, 3>;    // d_qk = d_v = 64, separate V tensor
using Cl64Cfg = TcCfg<1, 1, 64, 2, false, 1, 1, 3>;  // d_qk = d_v = 64, V = K

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D bf16 row-major [rows, cols] tensor, box [box_rows, 64 columns], 128-byte swizzle.
static bool make_map(CUtensorMap *m, const void *base, long long rows, int cols, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc || rows <= 0) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_tensor_map_bf16(CUtensorMap *m, const void *base, long long rows, int cols, int box_rows) {
    return make_map(m, base, rows, cols, box_rows);
}

// The same [rows, cols] bf16 tensor seen as [cols/64 chunks][rows][64 columns] (the chunk dimension
// is the outermost box dimension although its stride, 128 B, is the smallest), so that one copy of a
// box {64, box_rows, box_chunks} lands in shared memory as box_chunks consecutive [box_rows x 128 B]
// swizzled tiles - the layout the MMA descriptors expect - instead of one copy per chunk.
bool make_tensor_map_bf16_chunked(CUtensorMap *m, const void *base, long long rows, int cols, int box_rows,
                                  int box_chunks) {
    EncodeTiledFn enc = get_encode();
    if (!enc || rows <= 0 || cols % 64 != 0) return false;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace fdmla

#include "tc_fwd2.cuh"   // 2-CTA kernel for the MLA dimensions

namespace fdmla {

static std::atomic<int> g_prefer_single_cta{0};                // debugging / A-B switch
void tensor_prefer_single_cta(int on) { g_prefer_single_cta.store(on); }
bool tensor_single_cta_preferred() { return g_prefer_single_cta.load() != 0; }

template <class C>
static bool cfg_matches(const FwdProblem &p) {
    if (p.d_qk != C::D_QK || p.d_v != C::D_V) return false;
    if (C::SEPV != (p.V != nullptr)) return false;
    if (p.page_table && (p.page_size % C::T) != 0) return false;
    return true;
}

bool fwd_tensor_supported(const FwdProblem &p, int dtype) {
    if (dtype != FDMLA_BF16) return false;
    if (p.G <= 0 || p.R <= 0 || p.G > 65535 || p.num_splits > 65535) return false;
    const long long kv_rows = p.page_table ? (long long)p.num_pages * p.page_size : (long long)p.G * p.Skv;
    if (kv_rows <= 0 || kv_rows > 2147483647LL || (long long)p.G * p.R > 2147483647LL) return false;
    if ((reinterpret_cast<uintptr_t>(p.Q) | reinterpret_cast<uintptr_t>(p.K) | reinterpret_cast<uintptr_t>(p.V)) & 15)
        return false;
    if ((reinterpret_cast<uintptr_t>(p.O) | reinterpret_cast<uintptr_t>(p.O_part)) & 15) return false;
    return cfg_matches<MlaCfg>(p) || cfg_matches<OtfCfg>(p) || cfg_matches<Cl64Cfg>(p);
}

template <class C>
static int launch_cfg(const FwdProblem &p, cudaStream_t stream) {
    CUtensorMap tmQ, tmK, tmV;
    const long long kv_rows = p.page_table ? (long long)p.num_pages * p.page_size : (long long)p.G * p.Skv;
    if (!make_map(&tmQ, p.Q, (long long)p.G * p.R, p.d_qk, 128)) return FDMLA_ERR_CUDA;
    if (!make_map(&tmK, p.K, kv_rows, p.d_qk, C::T)) return FDMLA_ERR_CUDA;
    if (C::SEPV) {
        if (!make_map(&tmV, p.V, kv_rows, p.d_v, C::T)) return FDMLA_ERR_CUDA;
    } else {
        tmV = tmK;
    }
    auto kern = fwd_tc_kernel<C>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    if (C::CTAS_PER_SM > 1 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    dim3 grid(((p.R + 127) / 128) * C::VSPLIT, p.G, p.num_splits);
    kern<<<grid, TC_THREADS, C::SMEM_BYTES, stream>>>(p, tmQ, tmK, tmV);
    return check_launch();
}

int launch_fwd_tensor(const FwdProblem &p, int dtype, cudaStream_t stream) {
    if (!fwd_tensor_supported(p, dtype)) return FDMLA_ERR_UNSUPPORTED;
    if (!g_prefer_single_cta.load() && fwd_tensor2_supported(p, dtype)) return launch_fwd_tensor2(p, stream);
    if (cfg_matches<MlaCfg>(p)) return launch_cfg<MlaCfg>(p, stream);
    if (cfg_matches<OtfCfg>(p)) return launch_cfg<OtfCfg>(p, stream);
    return launch_cfg<Cl64Cfg>(p, stream);
}

int tensor_error_flag(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        int z = 0;
        cudaMemcpyToSymbol(g_tc_error, &z, sizeof(int));
    }
    return v;
}

}  // namespace fdmla
