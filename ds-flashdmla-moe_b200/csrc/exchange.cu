// Exchange and merge of the ranks' partial attention results in ONE kernel, over NVLink peer memory.
//
// Long-context decode splits every sequence's KV cache over the GPUs of a node; each rank attends its slice and holds
// a partial result per row - O (normalised, d_v floats), m (row maximum), l (row sum) - in one fp32 message
// [ O (rows x d_v) | m (rows) | l (rows) ].  Every rank needs the merged result.  The reference's MPI wrapper gathers K
// and V themselves with MPI_Allgatherv on the host (csrc/attention/fa2_fwd_mpi.cu:65-74) and runs the whole attention
// on every rank; the merge rule is the running update of csrc/attention/fa2_fwd.cu:93-111 applied across partials:
//     m = max_p m_p,   w_p = l_p exp(m_p - m),   l = sum_p w_p,   O = sum_p (w_p / l) O_p.
//
// Every rank owns an exchange buffer that its peers have mapped (CUDA IPC).  Per slot (two slots, used in turn):
//     [ world messages: the peers' partial rows for the row blocks this rank merges | one result area ]
// and behind the slots   [ data flags: world x GRID words | result flags: GRID words | step counters: GRID words ].
// One launch of exchange_merge_kernel on every rank does the step.  The grid is GRID thread blocks on every rank (all
// resident at once: 512 threads, no shared memory to speak of); block c stands for the same run of rows everywhere.
// Two forms.  All-gather form (up to four ranks): the block stores its rows of this rank's message into message [rank]
// of every peer's slot, flags every peer, waits for every peer's flag and merges its rows itself - one hop.  Owner form
// (more ranks): rank c mod world is the OWNER of run c; the partials travel to the owner only and the merged rows
// travel back, so a rank sends (world - 1) / world of its message plus its share of the results instead of
// world - 1 whole messages:
//   not the owner:  the block stores its rows of this rank's message into message [rank] of the owner's current slot
//                   (plain 16-byte stores to peer memory), fences at system scope and writes the step number into
//                   data flag [rank][c] of the owner (st.release.sys); then it waits for result flag [c] of its own
//                   buffer (ld.acquire.sys) and copies the merged rows from its own result area to O, m, l;
//   the owner:      the block waits until data flag [p][c] of its own buffer has reached the step number for every
//                   peer p, merges its rows (a warp per row: this rank's part straight from the message, the peers'
//                   parts from its own buffer, part by part in rank order), writes them to its own O, m, l and into
//                   the result area of every peer, fences, and writes the step number into result flag [c] of every peer.
// Every wait is bounded by a time limit on the global timer: a peer that never arrives sets error code 31 and the block
// returns without writing a result.  A block never waits for another block of its own GPU, and the owner of a run
// waits only for stores that its peers issue before they wait themselves, so nothing depends on the order in which
// blocks are scheduled.  The step number is a counter kept per block in the rank's own buffer (a CUDA graph replays
// the launch unchanged); the slot alternates with it: for a run of rows, a rank can be at most one step ahead of a peer
// (each needs the other's flag of step s to finish step s), so it writes slot (s + 1) & 1 while the peer may still read
// slot s & 1.  All ranks must launch the same sequence of steps on one exchange, each rank from one stream, as with a
// collective.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstdlib>

#include "common.cuh"

namespace fdmla {
namespace xch {

constexpr int GRID = 128, THREADS = 512, MAX_WORLD = 16;
enum { ERR_EXCHANGE_TIMEOUT = 31 };

__device__ int g_xch_error = 0;

struct Args {
    // The pieces of this rank's partial result that are still to be merged into its message (num_parts > 0: dense
    // [num_parts, rows, d_v], [num_parts, rows], [num_parts, rows]; parts with l <= 0 hold nothing), or nothing
    // (num_parts == 0: msg already holds the rank's partial result).
    const float *O_part, *m_part, *l_part;
    int num_parts;
    float *msg;                    // this rank's message
    float *bufs[MAX_WORLD];        // exchange buffer of every rank as mapped here; bufs[rank] is this rank's own
    int world, rank;
    long long rows;
    int d_v;
    size_t stride;                 // floats between messages of a slot (the message size rounded up to 16 bytes)
    void *O;
    float *m, *l;
    unsigned long long timeout_ns;
};

__host__ __device__ inline size_t message_stride(long long rows, int d_v) {
    return ((size_t)rows * (size_t)(d_v + 2) + 3) & ~(size_t)3;
}
__host__ __device__ inline size_t slot_floats(int world, size_t stride) { return ((size_t)world + 1) * stride; }
__host__ __device__ inline size_t flags_offset_floats(int world, size_t stride) { return 2 * slot_floats(world, stride); }

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// four consecutive output elements, the first on a 16-byte (fp32) / 8-byte (bf16) boundary
__device__ __forceinline__ void store4(float *dst, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16 *dst, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t *>(&lo);
    w.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(dst) = w;
}

// bounded wait of one thread until *flag has reached `step`
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, uint32_t step, unsigned long long timeout_ns) {
    const unsigned long long t0 = global_timer_ns();
    while ((int)(ld_acquire_sys(flag) - step) < 0) {
        if (global_timer_ns() - t0 > timeout_ns) return false;
        __nanosleep(64);
    }
    return true;
}

template <typename TO, bool GATHER>
__global__ void __launch_bounds__(THREADS) exchange_merge_kernel(const Args a) {
    const int c = blockIdx.x, tid = threadIdx.x, W = a.world;
    float *own = a.bufs[a.rank];
    const size_t flags_off = flags_offset_floats(W, a.stride);
    uint32_t *data_flags = reinterpret_cast<uint32_t *>(own + flags_off);       // [world][GRID]
    uint32_t *res_flags = data_flags + (size_t)W * GRID;                        // [GRID]
    uint32_t *steps = res_flags + GRID;                                         // [GRID]
    __shared__ uint32_t s_step;
    __shared__ int s_bad;
    if (tid == 0) {
        s_step = steps[c] + 1;
        steps[c] = s_step;
        s_bad = 0;
    }
    __syncthreads();
    const uint32_t step = s_step;
    const size_t slot_off = (size_t)(step & 1) * slot_floats(W, a.stride);
    const size_t res_off = slot_off + (size_t)W * a.stride;                      // the slot's result area
    const long long per = (a.rows + GRID - 1) / GRID;
    const long long r0 = (long long)c * per;
    const long long r1 = r0 + per < a.rows ? r0 + per : a.rows;
    const long long nr = r1 > r0 ? r1 - r0 : 0;
    const size_t o_m = (size_t)a.rows * a.d_v, o_l = o_m + (size_t)a.rows;       // offsets of m and l in a message / result area
    const int owner = GATHER ? a.rank : c % W;        // all-gather form: every rank merges every run itself
    TO *O = static_cast<TO *>(a.O);

    if (a.num_parts > 0) {
        // ---- 0. this block's rows of the rank's own pieces into its message: a warp per row, the arithmetic of the
        // merge kernel, piece by piece in order (lane q holds m and l of pieces q and q + 32) ---------------------------
        const int warp = tid >> 5, lane = tid & 31, P = a.num_parts;
        const size_t so = (size_t)a.rows * a.d_v, sml = (size_t)a.rows;
        for (long long r = r0 + warp; r < r1; r += THREADS / 32) {
            float m_q[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_q[2] = {0.f, 0.f};
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (lane + 32 * h < P) {
                    l_q[h] = a.l_part[(size_t)(lane + 32 * h) * sml + r];
                    m_q[h] = a.m_part[(size_t)(lane + 32 * h) * sml + r];
                }
            auto l_of = [&](int q) { return __shfl_sync(0xffffffffu, q < 32 ? l_q[0] : l_q[1], q & 31); };
            auto m_of = [&](int q) { return __shfl_sync(0xffffffffu, q < 32 ? m_q[0] : m_q[1], q & 31); };
            float mx = -CUDART_INF_F;
            for (int q = 0; q < P; ++q) {
                const float lp = l_of(q), mp = m_of(q);
                if (lp > 0.f) mx = fmaxf(mx, mp);
            }
            float ls = 0.f;
            for (int q = 0; q < P; ++q) {
                const float lp = l_of(q), mp = m_of(q);
                if (lp > 0.f) ls += lp * __expf(mp - mx);
            }
            const float inv = ls > 0.f ? 1.f / ls : 0.f;
            for (int c0 = 0; c0 < a.d_v; c0 += 512) {
                float acc[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
                for (int q = 0; q < P; ++q) {
                    const float lp = l_of(q), mp = m_of(q);
                    if (lp > 0.f) {
                        const float w = lp * __expf(mp - mx) * inv;
                        const float *src = a.O_part + (size_t)q * so + (size_t)r * a.d_v;
                        float4 v[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int col = c0 + (i * 32 + lane) * 4;
                            v[i] = col < a.d_v ? *reinterpret_cast<const float4 *>(src + col) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            acc[i][0] = fmaf(w, v[i].x, acc[i][0]); acc[i][1] = fmaf(w, v[i].y, acc[i][1]);
                            acc[i][2] = fmaf(w, v[i].z, acc[i][2]); acc[i][3] = fmaf(w, v[i].w, acc[i][3]);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int col = c0 + (i * 32 + lane) * 4;
                    if (col < a.d_v) store4(a.msg + (size_t)r * a.d_v + col, acc[i]);
                }
            }
            if (lane == 0) { a.msg[o_m + r] = mx; a.msg[o_l + r] = ls; }
        }
        __syncthreads();          // the rows are read back below by other threads of this block
    }

    if (GATHER) {
        // ---- this block's rows of this rank's message into every peer's buffer -------------------------------
        const float4 *src = reinterpret_cast<const float4 *>(a.msg + (size_t)r0 * a.d_v);
        const size_t dst_off = slot_off + (size_t)a.rank * a.stride;
        const long long n4 = nr * a.d_v / 4;
        for (long long i = tid; i < n4; i += THREADS) {
            const float4 v = __ldcg(src + i);
            for (int p = 0; p < W; ++p)
                if (p != a.rank) reinterpret_cast<float4 *>(a.bufs[p] + dst_off + (size_t)r0 * a.d_v)[i] = v;
        }
        for (long long i = tid; i < nr; i += THREADS) {
            const float mv = __ldcg(a.msg + o_m + r0 + i), lv = __ldcg(a.msg + o_l + r0 + i);
            for (int p = 0; p < W; ++p)
                if (p != a.rank) {
                    a.bufs[p][dst_off + o_m + r0 + i] = mv;
                    a.bufs[p][dst_off + o_l + r0 + i] = lv;
                }
        }
        __threadfence_system();
        __syncthreads();
        if (tid < W && tid != a.rank)
            st_release_sys(reinterpret_cast<uint32_t *>(a.bufs[tid] + flags_off) + (size_t)a.rank * GRID + c, step);
    } else if (owner != a.rank) {
        // ---- this block's rows of this rank's message to their owner -----------------------------------------
        float *dst = a.bufs[owner] + slot_off + (size_t)a.rank * a.stride;
        const float4 *src = reinterpret_cast<const float4 *>(a.msg + (size_t)r0 * a.d_v);
        float4 *dst4 = reinterpret_cast<float4 *>(dst + (size_t)r0 * a.d_v);
        const long long n4 = nr * a.d_v / 4;
        for (long long i = tid; i < n4; i += THREADS) dst4[i] = __ldcg(src + i);
        for (long long i = tid; i < nr; i += THREADS) {
            dst[o_m + r0 + i] = __ldcg(a.msg + o_m + r0 + i);
            dst[o_l + r0 + i] = __ldcg(a.msg + o_l + r0 + i);
        }
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            uint32_t *owner_flags = reinterpret_cast<uint32_t *>(a.bufs[owner] + flags_off);
            st_release_sys(owner_flags + (size_t)a.rank * GRID + c, step);
            // ---- until the owner has stored the merged rows here ----------------------------------------------
            if (!wait_flag(res_flags + c, step, a.timeout_ns)) {
                atomicCAS(&g_xch_error, 0, ERR_EXCHANGE_TIMEOUT);
                s_bad = 1;
            }
        }
        __syncthreads();
        if (s_bad) return;
        const float *res = own + res_off;
        const uint2 *rs = reinterpret_cast<const uint2 *>(reinterpret_cast<const TO *>(res) + (size_t)r0 * a.d_v);
        uint2 *od = reinterpret_cast<uint2 *>(O + (size_t)r0 * a.d_v);
        const long long n8 = nr * a.d_v * (long long)sizeof(TO) / 8;
        for (long long i = tid; i < n8; i += THREADS) od[i] = __ldcg(rs + i);
        for (long long i = tid; i < nr; i += THREADS) {
            a.m[r0 + i] = __ldcg(res + o_m + r0 + i);
            a.l[r0 + i] = __ldcg(res + o_l + r0 + i);
        }
        return;
    }

    // ---- the owner: until every peer's rows of this block have landed here ----------------------------------------
    if (tid < W && tid != a.rank && !wait_flag(data_flags + (size_t)tid * GRID + c, step, a.timeout_ns)) {
        atomicCAS(&g_xch_error, 0, ERR_EXCHANGE_TIMEOUT);
        s_bad = 1;
    }
    __syncthreads();
    if (s_bad) return;

    // ---- merge: a warp per row; the arithmetic of the merge kernel of the split-KV decode, part by part in rank order
    // (every lane runs the same sums, so the result does not depend on the number of lanes) ---------------------------
    const int warp = tid >> 5, lane = tid & 31;
    for (long long r = r0 + warp; r < r1; r += THREADS / 32) {
        // lane q holds m and l of part q
        float m_q = -CUDART_INF_F, l_q = 0.f;
        if (lane < W) {
            const float *part = lane == a.rank ? a.msg : own + slot_off + (size_t)lane * a.stride;
            l_q = __ldcg(part + o_l + r);
            m_q = __ldcg(part + o_m + r);
        }
        float mx = -CUDART_INF_F;
        for (int q = 0; q < W; ++q) {
            const float lp = __shfl_sync(0xffffffffu, l_q, q), mp = __shfl_sync(0xffffffffu, m_q, q);
            if (lp > 0.f) mx = fmaxf(mx, mp);
        }
        float ls = 0.f;
        for (int q = 0; q < W; ++q) {
            const float lp = __shfl_sync(0xffffffffu, l_q, q), mp = __shfl_sync(0xffffffffu, m_q, q);
            if (lp > 0.f) ls += lp * __expf(mp - mx);
        }
        const float inv = ls > 0.f ? 1.f / ls : 0.f;
        for (int c0 = 0; c0 < a.d_v; c0 += 512) {               // 4 x (32 lanes x 4 columns) per pass
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            for (int q = 0; q < W; ++q) {
                const float lp = __shfl_sync(0xffffffffu, l_q, q), mp = __shfl_sync(0xffffffffu, m_q, q);
                if (lp > 0.f) {
                    const float w = lp * __expf(mp - mx) * inv;
                    const float *src = (q == a.rank ? a.msg : own + slot_off + (size_t)q * a.stride) + (size_t)r * a.d_v;
                    float4 v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int col = c0 + (i * 32 + lane) * 4;
                        v[i] = col < a.d_v ? __ldcg(reinterpret_cast<const float4 *>(src + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[i][0] = fmaf(w, v[i].x, acc[i][0]); acc[i][1] = fmaf(w, v[i].y, acc[i][1]);
                        acc[i][2] = fmaf(w, v[i].z, acc[i][2]); acc[i][3] = fmaf(w, v[i].w, acc[i][3]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int col = c0 + (i * 32 + lane) * 4;
                if (col < a.d_v) {
                    store4(O + (size_t)r * a.d_v + col, acc[i]);
                    if (!GATHER)
                        for (int p = 0; p < W; ++p)
                            if (p != a.rank) store4(reinterpret_cast<TO *>(a.bufs[p] + res_off) + (size_t)r * a.d_v + col, acc[i]);
                }
            }
        }
        if (lane == 0) {
            a.m[r] = mx;
            a.l[r] = ls;
            for (int p = 0; !GATHER && p < W; ++p)
                if (p != a.rank) {
                    a.bufs[p][res_off + o_m + r] = mx;
                    a.bufs[p][res_off + o_l + r] = ls;
                }
        }
    }
    if (GATHER) return;
    __threadfence_system();
    __syncthreads();
    if (tid < W && tid != a.rank) {
        uint32_t *peer_res_flags = reinterpret_cast<uint32_t *>(a.bufs[tid] + flags_off) + (size_t)W * GRID;
        st_release_sys(peer_res_flags + c, step);
    }
}

}  // namespace xch

int exchange_error_flag(int reset) {
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, xch::g_xch_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(xch::g_xch_error, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return v;
}

size_t exchange_bytes(int world, long long rows, int d_v) {
    if (world < 1 || world > xch::MAX_WORLD || rows <= 0 || d_v <= 0 || (d_v & 3)) return 0;
    const size_t stride = xch::message_stride(rows, d_v);
    return (xch::flags_offset_floats(world, stride) + (size_t)world * xch::GRID + 2 * xch::GRID) * sizeof(float);
}

int launch_exchange_merge(const float *O_part, const float *m_part, const float *l_part, int num_parts, void *msg,
                          void *const *bufs, int world, int rank, long long rows, int d_v, void *O,
                          float *m, float *l, int out_dtype, int timeout_ms, cudaStream_t stream) {
    using namespace xch;
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || rows < 0 || d_v <= 0 || timeout_ms <= 0) return FDMLA_ERR_INVALID;
    if (rows == 0) return FDMLA_OK;
    if (!msg || !bufs || !O || !m || !l || num_parts < 0 || num_parts > 64) return FDMLA_ERR_INVALID;
    if (num_parts > 0 && (!O_part || !m_part || !l_part)) return FDMLA_ERR_INVALID;
    if (d_v & 3) return FDMLA_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(O_part) & 15) return FDMLA_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(msg) | reinterpret_cast<uintptr_t>(O)) & 15) return FDMLA_ERR_UNSUPPORTED;
    Args a{};
    a.O_part = O_part; a.m_part = m_part; a.l_part = l_part; a.num_parts = num_parts;
    a.msg = static_cast<float *>(msg);
    for (int p = 0; p < world; ++p) {
        if (!bufs[p] || (reinterpret_cast<uintptr_t>(bufs[p]) & 15)) return FDMLA_ERR_INVALID;
        a.bufs[p] = static_cast<float *>(bufs[p]);
    }
    a.world = world; a.rank = rank; a.rows = rows; a.d_v = d_v;
    a.stride = message_stride(rows, d_v);
    a.O = O; a.m = m; a.l = l;
    a.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    // up to four ranks: every rank sends its whole message to every other and merges everything itself (one hop); more:
    // the rows go to their owners and the merged rows come back (two hops, a fraction of the traffic).  Measured on
    // B=8, H=128 (2 MB messages) over NVLink: 2 ranks 0.160 / 0.175 ms per decode step (one hop / two hops), 4 ranks
    // 0.127 / 0.136, 8 ranks 0.124 / 0.117.
    static const int forced = [] { const char *e = getenv("FDMLA_EXCHANGE_GATHER"); return e && *e ? atoi(e) : -1; }();
    const bool gather = forced >= 0 ? forced != 0 : world <= 4;
    if (out_dtype == FDMLA_F32) {
        if (gather) exchange_merge_kernel<float, true><<<GRID, THREADS, 0, stream>>>(a);
        else exchange_merge_kernel<float, false><<<GRID, THREADS, 0, stream>>>(a);
    } else if (out_dtype == FDMLA_BF16) {
        if (gather) exchange_merge_kernel<__nv_bfloat16, true><<<GRID, THREADS, 0, stream>>>(a);
        else exchange_merge_kernel<__nv_bfloat16, false><<<GRID, THREADS, 0, stream>>>(a);
    } else {
        return FDMLA_ERR_INVALID;
    }
    return check_launch();
}

}  // namespace fdmla
