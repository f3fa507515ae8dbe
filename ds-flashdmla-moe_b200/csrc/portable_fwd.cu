// Portable (CUDA-core, fp32 math) Flash-DMLA forward: any dtype, any head
// dimensions up to d_qk <= 576 / d_v <= 512, dense or paged keys, causal or
// not, split-KV.  It is the kernel behind fp32 inputs and odd shapes; the
// tcgen05 kernels take over for the bf16 production shapes.
//
// The per-tile recurrence is the online softmax of the reference's
// csrc/attention/fa2_fwd.cu:88-128 (m_new, alpha, l_new), with the output kept
// un-normalised until the end instead of being renormalised every tile.
#include "common.cuh"

namespace fdmla {

constexpr int PF_THREADS = 128;  // 4 warps
constexpr int PF_ROWS = 16;      // query rows per block, 4 per warp
constexpr int PF_RW = 4;
constexpr int PF_TOK = 32;       // keys per tile, one per lane

__host__ __device__ inline int pf_ldk(int d_qk) {
    int d4 = (d_qk + 3) & ~3;
    return ((d4 / 4) & 1) ? d4 : d4 + 4;   // (ldk/4) odd: conflict-free 16-byte row reads
}

template <typename T, int NC>
__global__ void __launch_bounds__(PF_THREADS)
fwd_portable_kernel(const FwdProblem p) {
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.y, split = blockIdx.z;
    const int row0 = blockIdx.x * PF_ROWS;
    const int d_qk = p.d_qk, d_v = p.d_v;
    const int ldq = (d_qk + 3) & ~3;
    const int ldk = pf_ldk(d_qk);
    const bool sepV = (p.V != nullptr);

    long long *rowoff = reinterpret_cast<long long *>(smem);   // [32] pool/dense row of each key
    float *Qs = smem + 2 * PF_TOK;                        // [16][ldq]
    float *Ks = Qs + PF_ROWS * ldq;                      // [32][ldk] (+32 slack)
    float *Vs = sepV ? Ks + PF_TOK * ldk + 32 : Ks;      // [32][d_v] (+32 slack)
    const int ldvs = sepV ? d_v : ldk;

    const int seq = p.seqlens ? p.seqlens[g] : p.Skv;
    int w_lo = p.kv_begin > 0 ? p.kv_begin : 0;
    int w_hi = (p.kv_end >= 0 && p.kv_end < seq) ? p.kv_end : seq;
    int lo, hi;
    const int gran = p.page_table ? p.page_size : PF_TOK;
    split_window(w_lo, w_hi, gran, split, p.num_splits, &lo, &hi);

    // stage the block's query rows
    const T *Qg = static_cast<const T *>(p.Q) + ((size_t)g * p.R + row0) * d_qk;
    for (int idx = tid; idx < PF_ROWS * ldq; idx += PF_THREADS) {
        int r = idx / ldq, k = idx - r * ldq;
        float v = 0.f;
        if (row0 + r < p.R && k < d_qk) v = to_f32(Qg[(size_t)r * d_qk + k]);
        Qs[idx] = v;
    }

    // per-row visibility limits
    int upper[PF_RW];
    int block_hi = lo;
#pragma unroll
    for (int r = 0; r < PF_RW; ++r) upper[r] = lo;
    for (int r = 0; r < PF_ROWS; ++r) {
        int rr = row0 + r;
        int u = lo;
        if (rr < p.R) {
            int i = rr % p.Sq;
            long long vis = p.causal ? (long long)i + seq - p.Sq + 1 : seq;
            if (vis > seq) vis = seq;
            if (vis < 0) vis = 0;
            u = (int)(vis < hi ? vis : hi);
            if (u < lo) u = lo;
        }
        if (u > block_hi) block_hi = u;
        if ((r >> 2) == warp) upper[r & 3] = u;
    }

    float m_run[PF_RW], l_run[PF_RW], acc[PF_RW][NC];
#pragma unroll
    for (int r = 0; r < PF_RW; ++r) {
        m_run[r] = -CUDART_INF_F;
        l_run[r] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
    }

    const T *Kg = static_cast<const T *>(p.K);
    const T *Vg = static_cast<const T *>(p.V);

    for (int t0 = lo; t0 < block_hi; t0 += PF_TOK) {
        __syncthreads();   // previous tile fully consumed (also orders the Q staging)
        if (tid < PF_TOK) {
            int t = t0 + tid;
            long long off = -1;
            if (t < block_hi) {
                if (p.page_table) {
                    int lp = t / p.page_size;
                    int pg = (lp < p.max_pages) ? p.page_table[(size_t)g * p.max_pages + lp] : -1;
                    if (pg >= 0 && pg < p.num_pages) off = (long long)pg * p.page_size + (t - lp * p.page_size);
                } else {
                    off = (long long)g * p.Skv + t;
                }
            }
            rowoff[tid] = off;
        }
        __syncthreads();
        for (int idx = tid; idx < PF_TOK * ldk; idx += PF_THREADS) {
            int j = idx / ldk, k = idx - j * ldk;
            long long off = rowoff[j];
            float v = 0.f;
            if (off >= 0 && k < d_qk) v = to_f32(Kg[(size_t)off * d_qk + k]);
            Ks[idx] = v;
        }
        if (sepV) {
            for (int idx = tid; idx < PF_TOK * d_v; idx += PF_THREADS) {
                int j = idx / d_v, c = idx - j * d_v;
                long long off = rowoff[j];
                Vs[idx] = off >= 0 ? to_f32(Vg[(size_t)off * d_v + c]) : 0.f;
            }
        }
        __syncthreads();

        // scores: lane = key
        float s[PF_RW] = {0.f, 0.f, 0.f, 0.f};
        const float4 *k4 = reinterpret_cast<const float4 *>(Ks + lane * ldk);
        const float4 *q4 = reinterpret_cast<const float4 *>(Qs + (warp * PF_RW) * ldq);
        const int n4 = ldq >> 2;
        for (int k = 0; k < n4; ++k) {
            float4 kv = k4[k];
#pragma unroll
            for (int r = 0; r < PF_RW; ++r) {
                float4 qv = q4[r * n4 + k];
                s[r] = fmaf(qv.x, kv.x, s[r]);
                s[r] = fmaf(qv.y, kv.y, s[r]);
                s[r] = fmaf(qv.z, kv.z, s[r]);
                s[r] = fmaf(qv.w, kv.w, s[r]);
            }
        }
        float pr[PF_RW];
#pragma unroll
        for (int r = 0; r < PF_RW; ++r) {
            bool valid = (t0 + lane) < upper[r];
            float sv = valid ? s[r] * p.scale : -CUDART_INF_F;
            float m_new = fmaxf(m_run[r], warp_max(sv));
            float alpha = 1.f, pv = 0.f;
            if (m_new != -CUDART_INF_F) {
                alpha = (m_run[r] == -CUDART_INF_F) ? 0.f : __expf(m_run[r] - m_new);
                pv = valid ? __expf(sv - m_new) : 0.f;
            }
            l_run[r] = l_run[r] * alpha + warp_sum(pv);
            m_run[r] = m_new;
            pr[r] = pv;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[r][c] *= alpha;
        }
        // O += P V : lane owns columns lane + 32*c
        for (int j = 0; j < PF_TOK; ++j) {
            float pj[PF_RW];
#pragma unroll
            for (int r = 0; r < PF_RW; ++r) pj[r] = __shfl_sync(0xffffffffu, pr[r], j);
            const float *vr = Vs + j * ldvs + lane;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float vv = (lane + 32 * c < d_v) ? vr[32 * c] : 0.f;
#pragma unroll
                for (int r = 0; r < PF_RW; ++r) acc[r][c] = fmaf(pj[r], vv, acc[r][c]);
            }
        }
    }

    // epilogue
    const bool final_out = (p.num_splits == 1 && p.O != nullptr);
#pragma unroll
    for (int r = 0; r < PF_RW; ++r) {
        int rr = row0 + warp * PF_RW + r;
        if (rr >= p.R) continue;
        float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
        size_t grow = (size_t)g * p.R + rr;
        if (final_out) {
            T *o = static_cast<T *>(p.O) + grow * d_v;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                int col = lane + 32 * c;
                if (col < d_v) o[col] = from_f32<T>(acc[r][c] * inv);
            }
            if (lane == 0) { p.m[grow] = m_run[r]; p.l[grow] = l_run[r]; }
        } else {
            size_t prow = (size_t)split * p.G * p.R + grow;
            float *o = p.O_part + prow * d_v;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                int col = lane + 32 * c;
                if (col < d_v) o[col] = acc[r][c] * inv;
            }
            if (lane == 0) { p.m_part[prow] = m_run[r]; p.l_part[prow] = l_run[r]; }
        }
    }
}

template <typename T, int NC>
static int launch_pf(const FwdProblem &p, cudaStream_t stream) {
    const int ldq = (p.d_qk + 3) & ~3, ldk = pf_ldk(p.d_qk);
    size_t floats = (size_t)PF_ROWS * ldq + (size_t)PF_TOK * ldk + 32;
    if (p.V) floats += (size_t)PF_TOK * p.d_v + 32;
    size_t bytes = floats * sizeof(float) + PF_TOK * sizeof(long long);
    if (bytes > (size_t)kMaxSmemPerBlock) return FDMLA_ERR_UNSUPPORTED;
    auto kern = fwd_portable_kernel<T, NC>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    dim3 grid((p.R + PF_ROWS - 1) / PF_ROWS, p.G, p.num_splits);
    kern<<<grid, PF_THREADS, bytes, stream>>>(p);
    return check_launch();
}

template <typename T>
static int launch_pf_t(const FwdProblem &p, cudaStream_t stream) {
    int nc = (p.d_v + 31) / 32;
    if (nc <= 2) return launch_pf<T, 2>(p, stream);
    if (nc <= 4) return launch_pf<T, 4>(p, stream);
    if (nc <= 8) return launch_pf<T, 8>(p, stream);
    if (nc <= 16) return launch_pf<T, 16>(p, stream);
    return FDMLA_ERR_UNSUPPORTED;
}

int launch_fwd_portable(const FwdProblem &p, int dtype, cudaStream_t stream) {
    if (p.G <= 0 || p.R <= 0) return FDMLA_OK;
    if (p.G > 65535 || p.num_splits > 65535) return FDMLA_ERR_UNSUPPORTED;
    if (dtype == FDMLA_F32) return launch_pf_t<float>(p, stream);
    if (dtype == FDMLA_BF16) return launch_pf_t<__nv_bfloat16>(p, stream);
    return FDMLA_ERR_INVALID;
}

// ---------------------------------------------------------------------------
// Log-sum-exp merge of partials: one warp per row, rows strided over a grid that
// fills the GPU once.
// m = max m_p; w_p = l_p exp(m_p - m); l = sum w_p; O = sum w_p O_p / l
// (the running update of fa2_fwd.cu:93-111 applied across partial results).
// Parts with l_p <= 0 hold nothing and are not read.  l_part[0][row] < 0 marks a
// row whose final O, m, l have already been written (balanced decode schedule):
// it is left alone.
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
merge_kernel(const float *__restrict__ O_part, const float *__restrict__ m_part,
             const float *__restrict__ l_part, TO *__restrict__ O, float *__restrict__ m,
             float *__restrict__ l, long long rows, int d_v, int P, size_t so, size_t sml, bool vec) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        if (l_part[r] < 0.f) continue;
        float mx = -CUDART_INF_F;
        for (int q = lane; q < P; q += 32)
            if (l_part[q * sml + r] > 0.f) mx = fmaxf(mx, m_part[q * sml + r]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float ls = 0.f;
        for (int q = lane; q < P; q += 32) {
            const float lp = l_part[q * sml + r];
            if (lp > 0.f) ls += lp * __expf(m_part[q * sml + r] - mx);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
        const float inv = ls > 0.f ? 1.f / ls : 0.f;
        for (int c0 = 0; c0 < d_v; c0 += 128) {
            const int c = c0 + lane * 4;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < P; ++q) {
                const float lp = l_part[q * sml + r];         // same address in every lane
                if (lp > 0.f) {
                    const float w = lp * __expf(m_part[q * sml + r] - mx) * inv;
                    const float *src = O_part + (size_t)q * so + (size_t)r * d_v;
                    if (vec && c + 3 < d_v) {
                        const float4 v = *reinterpret_cast<const float4 *>(src + c);
                        acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
                        acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
                    } else {
                        for (int e = 0; e < 4; ++e)
                            if (c + e < d_v) acc[e] = fmaf(w, src[c + e], acc[e]);
                    }
                }
            }
            for (int e = 0; e < 4; ++e)
                if (c + e < d_v) O[(size_t)r * d_v + c + e] = from_f32<TO>(acc[e]);
        }
        if (lane == 0) { m[r] = mx; l[r] = ls; }
    }
}

// The same merge with one block per row (few rows, many parts: more loads in flight per row).
template <typename TO>
__global__ void __launch_bounds__(128)
merge_row_block_kernel(const float *__restrict__ O_part, const float *__restrict__ m_part,
                       const float *__restrict__ l_part, TO *__restrict__ O, float *__restrict__ m,
                       float *__restrict__ l, long long rows, int d_v, int P, size_t so, size_t sml, bool vec) {
    const long long r = blockIdx.x;
    if (l_part[r] < 0.f) return;
    float mx = -CUDART_INF_F;
    for (int q = 0; q < P; ++q)
        if (l_part[q * sml + r] > 0.f) mx = fmaxf(mx, m_part[q * sml + r]);
    float ls = 0.f;
    for (int q = 0; q < P; ++q) {
        const float lp = l_part[q * sml + r];
        if (lp > 0.f) ls += lp * __expf(m_part[q * sml + r] - mx);
    }
    const float inv = ls > 0.f ? 1.f / ls : 0.f;
    for (int c = threadIdx.x * 4; c < d_v; c += 512) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int q = 0; q < P; ++q) {
            const float lp = l_part[q * sml + r];
            if (lp > 0.f) {
                const float w = lp * __expf(m_part[q * sml + r] - mx) * inv;
                const float *src = O_part + (size_t)q * so + (size_t)r * d_v;
                if (vec && c + 3 < d_v) {
                    const float4 v = *reinterpret_cast<const float4 *>(src + c);
                    acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
                    acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
                } else {
                    for (int e = 0; e < 4; ++e)
                        if (c + e < d_v) acc[e] = fmaf(w, src[c + e], acc[e]);
                }
            }
        }
        for (int e = 0; e < 4; ++e)
            if (c + e < d_v) O[(size_t)r * d_v + c + e] = from_f32<TO>(acc[e]);
    }
    if (threadIdx.x == 0) { m[r] = mx; l[r] = ls; }
}

// part_stride_o / part_stride_ml: elements between consecutive parts of O_part and of m_part / l_part
// (rows * d_v and rows for the dense [num_parts, rows, ...] layout).
int launch_merge_strided(const float *O_part, const float *m_part, const float *l_part, void *O,
                         float *m, float *l, long long rows, int d_v, int num_parts, size_t part_stride_o,
                         size_t part_stride_ml, int out_dtype, cudaStream_t stream) {
    if (rows <= 0) return FDMLA_OK;
    // 16-byte loads of O_part only where every part's rows start on a 16-byte boundary (gathered messages of an odd
    // number of rows do not)
    const bool vec = (d_v & 3) == 0 && (part_stride_o & 3) == 0 && (reinterpret_cast<uintptr_t>(O_part) & 15) == 0;
    if (rows <= 4096) {      // a block per row keeps more of the GPU busy than a warp per row would
        if (out_dtype == FDMLA_F32)
            merge_row_block_kernel<float><<<(unsigned)rows, 128, 0, stream>>>(O_part, m_part, l_part, static_cast<float *>(O), m, l,
                                                                               rows, d_v, num_parts, part_stride_o, part_stride_ml, vec);
        else if (out_dtype == FDMLA_BF16)
            merge_row_block_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, stream>>>(
                O_part, m_part, l_part, static_cast<__nv_bfloat16 *>(O), m, l, rows, d_v, num_parts, part_stride_o, part_stride_ml, vec);
        else
            return FDMLA_ERR_INVALID;
        return check_launch();
    }
    const long long want = (rows + 7) / 8;
    const unsigned grid = (unsigned)(want < 8LL * kNumSMs ? want : 8LL * kNumSMs);
    if (out_dtype == FDMLA_F32)
        merge_kernel<float><<<grid, 256, 0, stream>>>(O_part, m_part, l_part, static_cast<float *>(O), m, l, rows,
                                                      d_v, num_parts, part_stride_o, part_stride_ml, vec);
    else if (out_dtype == FDMLA_BF16)
        merge_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(O_part, m_part, l_part, static_cast<__nv_bfloat16 *>(O),
                                                             m, l, rows, d_v, num_parts, part_stride_o, part_stride_ml, vec);
    else
        return FDMLA_ERR_INVALID;
    return check_launch();
}

int launch_merge(const float *O_part, const float *m_part, const float *l_part, void *O,
                 float *m, float *l, long long rows, int d_v, int num_parts, int out_dtype,
                 cudaStream_t stream) {
    return launch_merge_strided(O_part, m_part, l_part, O, m, l, rows, d_v, num_parts, (size_t)rows * d_v, (size_t)rows,
                                out_dtype, stream);
}

// ---------------------------------------------------------------------------
// Dense projection Y[rows, d_out] = X[rows, d_in] * W   (W [d_in, d_out]), or
// with w_transposed: Y = X * W^T (W [d_out, d_in]).  fp32 accumulation.
// Block = 256 threads computes 32 rows; W is staged in shared memory as
// [d_in][d_out] fp32.  Used for K_lat = K*WK, V_lat = V*WV and, in the
// backward, dK = dK_lat*WK^T.
// ---------------------------------------------------------------------------
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256)
project_kernel(const TI *__restrict__ X, const TW *__restrict__ W, TO *__restrict__ Y,
               long long rows, int d_in, int d_out, int w_transposed) {
    extern __shared__ __align__(16) float smem[];
    float *Ws = smem;                       // [d_in][d_out]
    float *Xs = Ws + (size_t)d_in * d_out;  // [32][d_in + 1]
    const int tid = threadIdx.x;
    for (int idx = tid; idx < d_in * d_out; idx += 256) {
        int k = idx / d_out, n = idx - k * d_out;
        Ws[idx] = to_f32(w_transposed ? W[(size_t)n * d_in + k] : W[idx]);
    }
    const long long r0 = (long long)blockIdx.x * 32;
    const int ldx = d_in + 1;
    for (int idx = tid; idx < 32 * d_in; idx += 256) {
        int r = idx / d_in, k = idx - r * d_in;
        Xs[r * ldx + k] = (r0 + r < rows) ? to_f32(X[(size_t)(r0 + r) * d_in + k]) : 0.f;
    }
    __syncthreads();
    const int r = tid >> 3, cg = tid & 7;   // 32 rows x 8 column groups
    for (int n0 = cg; n0 < d_out; n0 += 64) {
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.f;
        for (int k = 0; k < d_in; ++k) {
            float x = Xs[r * ldx + k];
            const float *w = Ws + (size_t)k * d_out + n0;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (n0 + 8 * c < d_out) acc[c] = fmaf(x, w[8 * c], acc[c]);
        }
        if (r0 + r < rows) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (n0 + 8 * c < d_out) Y[(size_t)(r0 + r) * d_out + n0 + 8 * c] = from_f32<TO>(acc[c]);
        }
    }
}

template <typename TI, typename TW, typename TO>
static int launch_project_t(const void *X, const void *W, void *Y, long long rows, int d_in,
                            int d_out, int w_transposed, cudaStream_t stream) {
    size_t bytes = ((size_t)d_in * d_out + 32 * (size_t)(d_in + 1)) * sizeof(float);
    if (bytes > (size_t)kMaxSmemPerBlock) return FDMLA_ERR_UNSUPPORTED;
    auto kern = project_kernel<TI, TW, TO>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    long long blocks = (rows + 31) / 32;
    if (blocks > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    kern<<<(unsigned)blocks, 256, bytes, stream>>>(static_cast<const TI *>(X), static_cast<const TW *>(W),
                                                  static_cast<TO *>(Y), rows, d_in, d_out, w_transposed);
    return check_launch();
}

// x_f32 != 0: X is fp32 whatever `dtype` says (gradient workspaces); W and Y are `dtype`.
int launch_project(const void *X, const void *W, void *Y, long long rows, int d_in, int d_out,
                   int w_transposed, int x_f32, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FDMLA_OK;
    using bf = __nv_bfloat16;
    if (dtype == FDMLA_BF16 && tensor_kernels_allowed()) {
        const int rc = launch_project_tensor(X, W, Y, rows, d_in, d_out, w_transposed, x_f32, stream);
        if (rc != FDMLA_ERR_UNSUPPORTED) return rc;
    }
    if (dtype == FDMLA_F32)
        return launch_project_t<float, float, float>(X, W, Y, rows, d_in, d_out, w_transposed, stream);
    if (dtype == FDMLA_BF16 && x_f32)
        return launch_project_t<float, bf, bf>(X, W, Y, rows, d_in, d_out, w_transposed, stream);
    if (dtype == FDMLA_BF16)
        return launch_project_t<bf, bf, bf>(X, W, Y, rows, d_in, d_out, w_transposed, stream);
    return FDMLA_ERR_INVALID;
}

}  // namespace fdmla
