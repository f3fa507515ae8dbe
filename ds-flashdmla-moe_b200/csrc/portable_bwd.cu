// Portable (CUDA-core, fp32 math) Flash-DMLA backward.  P is recomputed from
// the saved row statistics, gradients are produced by owner-computes kernels
// (one for dQ, one for dK_lat/dV_lat), so nothing is accumulated with atomics
// and results are deterministic.
//
// Formulas follow the reference's csrc/attention/fa2_bwd.cu:
//   delta_i = sum_j P_ij (V_j . dO_i)         (:198-216)  == rowsum(dO o O)
//   dS_ij   = P_ij (dP_ij - delta_i)          (:234)
//   dK_j   += dS_ij q_i                       (:252-254)
//   dV_j   += P_ij dO_i                       (:259-272)
//   dQ_i   += dS_ij k_j                       (:293-309)
// with the softmax scale the reference leaves out applied to dQ and dK.
#include "common.cuh"

namespace fdmla {

__host__ __device__ inline int pb_ld(int d) {
    int d4 = (d + 3) & ~3;
    return ((d4 / 4) & 1) ? d4 : d4 + 4;
}

// D[row] = sum_c dO[row][c] * O[row][c]; one warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
bwd_delta_kernel(const T *__restrict__ O, const T *__restrict__ dO, float *__restrict__ D,
                 long long rows, int d_v) {
    long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    float acc = 0.f;
    for (int c = lane; c < d_v; c += 32)
        acc = fmaf(to_f32(O[(size_t)row * d_v + c]), to_f32(dO[(size_t)row * d_v + c]), acc);
    acc = warp_sum(acc);
    if (lane == 0) D[row] = acc;
}

constexpr int PB_THREADS = 128;
constexpr int PB_OWN = 16;   // rows (dQ kernel) or keys (dKV kernel) owned per block, 4 per warp
constexpr int PB_RW = 4;
constexpr int PB_TILE = 32;  // streamed keys (dQ kernel) or queries (dKV kernel), one per lane

__device__ __forceinline__ void dot4(const float *own, int ld_own, const float *strm, int n4,
                                     float (&s)[PB_RW]) {
    const float4 *a4 = reinterpret_cast<const float4 *>(strm);
    const float4 *o4 = reinterpret_cast<const float4 *>(own);
    const int ldo4 = ld_own >> 2;
    for (int k = 0; k < n4; ++k) {
        float4 a = a4[k];
#pragma unroll
        for (int r = 0; r < PB_RW; ++r) {
            float4 b = o4[r * ldo4 + k];
            s[r] = fmaf(a.x, b.x, s[r]);
            s[r] = fmaf(a.y, b.y, s[r]);
            s[r] = fmaf(a.z, b.z, s[r]);
            s[r] = fmaf(a.w, b.w, s[r]);
        }
    }
}

// dQ: block owns 16 query rows, streams key tiles.
template <typename T, int NCQ>
__global__ void __launch_bounds__(PB_THREADS)
bwd_dq_kernel(const BwdProblem p) {
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.y, row0 = blockIdx.x * PB_OWN;
    const int d_qk = p.d_qk, d_v = p.d_v;
    const int ldq = (d_qk + 3) & ~3, ldo = (d_v + 3) & ~3;
    const int ldk = pb_ld(d_qk), ldv = pb_ld(d_v);
    const bool sepV = p.V != nullptr;
    float *Qs = smem;                       // [16][ldq]
    float *dOs = Qs + PB_OWN * ldq;         // [16][ldo]
    float *Ks = dOs + PB_OWN * ldo;         // [32][ldk] + 32
    float *Vs = sepV ? Ks + PB_TILE * ldk + 32 : Ks;
    const int ldvs = sepV ? ldv : ldk;

    const T *Qg = static_cast<const T *>(p.Q) + ((size_t)g * p.R + row0) * d_qk;
    const T *dOg = static_cast<const T *>(p.dO) + ((size_t)g * p.R + row0) * d_v;
    for (int idx = tid; idx < PB_OWN * ldq; idx += PB_THREADS) {
        int r = idx / ldq, k = idx - r * ldq;
        Qs[idx] = (row0 + r < p.R && k < d_qk) ? to_f32(Qg[(size_t)r * d_qk + k]) : 0.f;
    }
    for (int idx = tid; idx < PB_OWN * ldo; idx += PB_THREADS) {
        int r = idx / ldo, k = idx - r * ldo;
        dOs[idx] = (row0 + r < p.R && k < d_v) ? to_f32(dOg[(size_t)r * d_v + k]) : 0.f;
    }

    int upper[PB_RW];
    float m_r[PB_RW], linv[PB_RW], D_r[PB_RW];
    int block_hi = 0;
    for (int r = 0; r < PB_OWN; ++r) {
        int rr = row0 + r, u = 0;
        if (rr < p.R) {
            int i = rr % p.Sq;
            long long vis = p.causal ? (long long)i + p.Skv - p.Sq + 1 : p.Skv;
            if (vis > p.Skv) vis = p.Skv;
            if (vis < 0) vis = 0;
            u = (int)vis;
        }
        if (u > block_hi) block_hi = u;
        if ((r >> 2) == warp) {
            upper[r & 3] = u;
            size_t grow = (size_t)g * p.R + (rr < p.R ? rr : 0);
            float lv = rr < p.R ? p.l[grow] : 0.f;
            m_r[r & 3] = rr < p.R ? p.m[grow] : 0.f;
            linv[r & 3] = lv > 0.f ? 1.f / lv : 0.f;
            D_r[r & 3] = rr < p.R ? p.D[grow] : 0.f;
            if (!(lv > 0.f)) upper[r & 3] = 0;
        }
    }
    float acc[PB_RW][NCQ];
#pragma unroll
    for (int r = 0; r < PB_RW; ++r)
#pragma unroll
        for (int c = 0; c < NCQ; ++c) acc[r][c] = 0.f;

    const T *Kg = static_cast<const T *>(p.K) + (size_t)g * p.Skv * d_qk;
    const T *Vg = sepV ? static_cast<const T *>(p.V) + (size_t)g * p.Skv * d_v : nullptr;
    for (int t0 = 0; t0 < block_hi; t0 += PB_TILE) {
        __syncthreads();
        for (int idx = tid; idx < PB_TILE * ldk; idx += PB_THREADS) {
            int j = idx / ldk, k = idx - j * ldk;
            Ks[idx] = (t0 + j < p.Skv && k < d_qk) ? to_f32(Kg[(size_t)(t0 + j) * d_qk + k]) : 0.f;
        }
        if (sepV)
            for (int idx = tid; idx < PB_TILE * ldv; idx += PB_THREADS) {
                int j = idx / ldv, k = idx - j * ldv;
                Vs[idx] = (t0 + j < p.Skv && k < d_v) ? to_f32(Vg[(size_t)(t0 + j) * d_v + k]) : 0.f;
            }
        __syncthreads();
        float s[PB_RW] = {0.f, 0.f, 0.f, 0.f}, dp[PB_RW] = {0.f, 0.f, 0.f, 0.f};
        dot4(Qs + warp * PB_RW * ldq, ldq, Ks + lane * ldk, ldq >> 2, s);
        dot4(dOs + warp * PB_RW * ldo, ldo, Vs + lane * ldvs, ldo >> 2, dp);
        float ds[PB_RW];
#pragma unroll
        for (int r = 0; r < PB_RW; ++r) {
            bool valid = (t0 + lane) < upper[r];
            float pv = valid ? __expf(s[r] * p.scale - m_r[r]) * linv[r] : 0.f;
            ds[r] = pv * (dp[r] - D_r[r]) * p.scale;
        }
        for (int j = 0; j < PB_TILE; ++j) {
            float dj[PB_RW];
#pragma unroll
            for (int r = 0; r < PB_RW; ++r) dj[r] = __shfl_sync(0xffffffffu, ds[r], j);
            const float *kr = Ks + j * ldk + lane;
#pragma unroll
            for (int c = 0; c < NCQ; ++c) {
                float kv = (lane + 32 * c < d_qk) ? kr[32 * c] : 0.f;
#pragma unroll
                for (int r = 0; r < PB_RW; ++r) acc[r][c] = fmaf(dj[r], kv, acc[r][c]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < PB_RW; ++r) {
        int rr = row0 + warp * PB_RW + r;
        if (rr >= p.R) continue;
        T *o = static_cast<T *>(p.dQ) + ((size_t)g * p.R + rr) * d_qk;
#pragma unroll
        for (int c = 0; c < NCQ; ++c) {
            int col = lane + 32 * c;
            if (col < d_qk) o[col] = from_f32<T>(acc[r][c]);
        }
    }
}

// dK_lat / dV_lat: block owns 16 keys of group g, streams query tiles of every
// head of the group.
template <typename T, typename TG, int NCQ, int NCV>
__global__ void __launch_bounds__(PB_THREADS)
bwd_dkv_kernel(const BwdProblem p) {
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.y, key0 = blockIdx.x * PB_OWN;
    const int d_qk = p.d_qk, d_v = p.d_v;
    const int ldq = (d_qk + 3) & ~3, ldo = (d_v + 3) & ~3;   // owned rows (broadcast reads)
    const int ldk = pb_ld(d_qk), ldv = pb_ld(d_v);           // streamed rows (lane-strided reads)
    const bool sepV = p.V != nullptr;
    float *Kown = smem;                                       // [16][ldq]
    float *Vown = sepV ? Kown + PB_OWN * ldq : Kown;          // [16][ldo] (or alias, stride ldq)
    const int ldvo = sepV ? ldo : ldq;
    float *Qs = Kown + PB_OWN * ldq + (sepV ? PB_OWN * ldo : 0);   // [32][ldk] + 32
    float *dOs = Qs + PB_TILE * ldk + 32;                     // [32][ldv] + 32

    const T *Kg = static_cast<const T *>(p.K) + (size_t)g * p.Skv * d_qk;
    for (int idx = tid; idx < PB_OWN * ldq; idx += PB_THREADS) {
        int r = idx / ldq, k = idx - r * ldq;
        Kown[idx] = (key0 + r < p.Skv && k < d_qk) ? to_f32(Kg[(size_t)(key0 + r) * d_qk + k]) : 0.f;
    }
    if (sepV) {
        const T *Vg = static_cast<const T *>(p.V) + (size_t)g * p.Skv * d_v;
        for (int idx = tid; idx < PB_OWN * ldo; idx += PB_THREADS) {
            int r = idx / ldo, k = idx - r * ldo;
            Vown[idx] = (key0 + r < p.Skv && k < d_v) ? to_f32(Vg[(size_t)(key0 + r) * d_v + k]) : 0.f;
        }
    }
    float accK[PB_RW][NCQ], accV[PB_RW][NCV];
#pragma unroll
    for (int r = 0; r < PB_RW; ++r) {
#pragma unroll
        for (int c = 0; c < NCQ; ++c) accK[r][c] = 0.f;
#pragma unroll
        for (int c = 0; c < NCV; ++c) accV[r][c] = 0.f;
    }
    const int Hg = p.R / p.Sq;
    const int shift = p.Skv - p.Sq;   // key j visible to query i iff j <= i + shift
    // first query that can see the block's first key
    int i_begin = 0;
    if (p.causal) { i_begin = key0 - shift; if (i_begin < 0) i_begin = 0; }
    i_begin = (i_begin / PB_TILE) * PB_TILE;

    for (int h = 0; h < Hg; ++h) {
        const size_t rbase = (size_t)g * p.R + (size_t)h * p.Sq;
        const T *Qg = static_cast<const T *>(p.Q) + rbase * d_qk;
        const T *dOg = static_cast<const T *>(p.dO) + rbase * d_v;
        for (int i0 = i_begin; i0 < p.Sq; i0 += PB_TILE) {
            __syncthreads();
            for (int idx = tid; idx < PB_TILE * ldk; idx += PB_THREADS) {
                int j = idx / ldk, k = idx - j * ldk;
                Qs[idx] = (i0 + j < p.Sq && k < d_qk) ? to_f32(Qg[(size_t)(i0 + j) * d_qk + k]) : 0.f;
            }
            for (int idx = tid; idx < PB_TILE * ldv; idx += PB_THREADS) {
                int j = idx / ldv, k = idx - j * ldv;
                dOs[idx] = (i0 + j < p.Sq && k < d_v) ? to_f32(dOg[(size_t)(i0 + j) * d_v + k]) : 0.f;
            }
            __syncthreads();
            const int i = i0 + lane;
            const bool qvalid = i < p.Sq;
            float mi = 0.f, li = 0.f, Di = 0.f;
            if (qvalid) { mi = p.m[rbase + i]; li = p.l[rbase + i]; Di = p.D[rbase + i]; }
            const float linv = li > 0.f ? 1.f / li : 0.f;
            float s[PB_RW] = {0.f, 0.f, 0.f, 0.f}, dp[PB_RW] = {0.f, 0.f, 0.f, 0.f};
            dot4(Kown + warp * PB_RW * ldq, ldq, Qs + lane * ldk, ldq >> 2, s);
            dot4(Vown + warp * PB_RW * ldvo, ldvo, dOs + lane * ldv, ldo >> 2, dp);
            float pv[PB_RW], ds[PB_RW];
#pragma unroll
            for (int r = 0; r < PB_RW; ++r) {
                int j = key0 + warp * PB_RW + r;
                bool valid = qvalid && li > 0.f && j < p.Skv && (!p.causal || j <= i + shift);
                pv[r] = valid ? __expf(s[r] * p.scale - mi) * linv : 0.f;
                ds[r] = pv[r] * (dp[r] - Di) * p.scale;
            }
            for (int q = 0; q < PB_TILE; ++q) {
                float dj[PB_RW], pj[PB_RW];
#pragma unroll
                for (int r = 0; r < PB_RW; ++r) {
                    dj[r] = __shfl_sync(0xffffffffu, ds[r], q);
                    pj[r] = __shfl_sync(0xffffffffu, pv[r], q);
                }
                const float *qr = Qs + q * ldk + lane;
#pragma unroll
                for (int c = 0; c < NCQ; ++c) {
                    float x = (lane + 32 * c < d_qk) ? qr[32 * c] : 0.f;
#pragma unroll
                    for (int r = 0; r < PB_RW; ++r) accK[r][c] = fmaf(dj[r], x, accK[r][c]);
                }
                const float *dr = dOs + q * ldv + lane;
#pragma unroll
                for (int c = 0; c < NCV; ++c) {
                    float x = (lane + 32 * c < d_v) ? dr[32 * c] : 0.f;
#pragma unroll
                    for (int r = 0; r < PB_RW; ++r) accV[r][c] = fmaf(pj[r], x, accV[r][c]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < PB_RW; ++r) {
        int j = key0 + warp * PB_RW + r;
        if (j >= p.Skv) continue;
        TG *ok = static_cast<TG *>(p.dK) + ((size_t)g * p.Skv + j) * d_qk;
        if (!sepV) {
#pragma unroll
            for (int c = 0; c < NCV; ++c)
                if (c < NCQ && lane + 32 * c < d_v) accK[r][c] += accV[r][c];
        } else {
            TG *ov = static_cast<TG *>(p.dV) + ((size_t)g * p.Skv + j) * d_v;
#pragma unroll
            for (int c = 0; c < NCV; ++c) {
                int col = lane + 32 * c;
                if (col < d_v) ov[col] = from_f32<TG>(accV[r][c]);
            }
        }
#pragma unroll
        for (int c = 0; c < NCQ; ++c) {
            int col = lane + 32 * c;
            if (col < d_qk) ok[col] = from_f32<TG>(accK[r][c]);
        }
    }
}

template <typename T, int NCQ>
static int launch_dq(const BwdProblem &p, cudaStream_t stream) {
    const int ldq = (p.d_qk + 3) & ~3, ldo = (p.d_v + 3) & ~3;
    size_t floats = (size_t)PB_OWN * ldq + (size_t)PB_OWN * ldo + (size_t)PB_TILE * pb_ld(p.d_qk) + 32;
    if (p.V) floats += (size_t)PB_TILE * pb_ld(p.d_v) + 32;
    size_t bytes = floats * sizeof(float);
    if (bytes > (size_t)kMaxSmemPerBlock) return FDMLA_ERR_UNSUPPORTED;
    auto kern = bwd_dq_kernel<T, NCQ>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    dim3 grid((p.R + PB_OWN - 1) / PB_OWN, p.G);
    kern<<<grid, PB_THREADS, bytes, stream>>>(p);
    return check_launch();
}

template <typename T, typename TG, int NCQ, int NCV>
static int launch_dkv(const BwdProblem &p, cudaStream_t stream) {
    const int ldq = (p.d_qk + 3) & ~3, ldo = (p.d_v + 3) & ~3;
    size_t floats = (size_t)PB_OWN * ldq + (p.V ? (size_t)PB_OWN * ldo : 0) +
                    (size_t)PB_TILE * pb_ld(p.d_qk) + 32 + (size_t)PB_TILE * pb_ld(p.d_v) + 32;
    size_t bytes = floats * sizeof(float);
    if (bytes > (size_t)kMaxSmemPerBlock) return FDMLA_ERR_UNSUPPORTED;
    auto kern = bwd_dkv_kernel<T, TG, NCQ, NCV>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    dim3 grid((p.Skv + PB_OWN - 1) / PB_OWN, p.G);
    kern<<<grid, PB_THREADS, bytes, stream>>>(p);
    return check_launch();
}

template <typename T, typename TG>
static int launch_bwd_t(const BwdProblem &p, cudaStream_t stream) {
    long long rows = (long long)p.G * p.R;
    if (rows <= 0 || p.Skv <= 0) return FDMLA_OK;
    if (p.G > 65535) return FDMLA_ERR_UNSUPPORTED;
    long long nblk = (rows + 7) / 8;
    if (nblk > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    bwd_delta_kernel<T><<<(unsigned)nblk, 256, 0, stream>>>(static_cast<const T *>(p.O),
                                                           static_cast<const T *>(p.dO), p.D, rows, p.d_v);
    int st = check_launch();
    if (st) return st;
    const int ncq = (p.d_qk + 31) / 32, ncv = (p.d_v + 31) / 32;
    if (ncq <= 2 && ncv <= 2) {
        st = launch_dq<T, 2>(p, stream);
        if (st) return st;
        return launch_dkv<T, TG, 2, 2>(p, stream);
    }
    if (ncq <= 4 && ncv <= 4) {
        st = launch_dq<T, 4>(p, stream);
        if (st) return st;
        return launch_dkv<T, TG, 4, 4>(p, stream);
    }
    if (ncq <= 8 && ncv <= 8) {
        st = launch_dq<T, 8>(p, stream);
        if (st) return st;
        return launch_dkv<T, TG, 8, 8>(p, stream);
    }
    if (ncq <= 18 && ncv <= 16) {
        st = launch_dq<T, 18>(p, stream);
        if (st) return st;
        return launch_dkv<T, TG, 18, 16>(p, stream);
    }
    return FDMLA_ERR_UNSUPPORTED;
}

int launch_bwd_delta(const BwdProblem &p, int dtype, cudaStream_t stream) {
    const long long rows = (long long)p.G * p.R;
    if (rows <= 0) return FDMLA_OK;
    const long long nblk = (rows + 7) / 8;
    if (nblk > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    if (dtype == FDMLA_F32)
        bwd_delta_kernel<float><<<(unsigned)nblk, 256, 0, stream>>>(static_cast<const float *>(p.O),
                                                                   static_cast<const float *>(p.dO), p.D, rows, p.d_v);
    else if (dtype == FDMLA_BF16)
        bwd_delta_kernel<__nv_bfloat16><<<(unsigned)nblk, 256, 0, stream>>>(
            static_cast<const __nv_bfloat16 *>(p.O), static_cast<const __nv_bfloat16 *>(p.dO), p.D, rows, p.d_v);
    else
        return FDMLA_ERR_INVALID;
    return check_launch();
}

// grads_f32: dK/dV are written as fp32 (latent-gradient workspaces of the
// on-the-fly mode) instead of `dtype`.
int launch_bwd_portable(const BwdProblem &p, int dtype, int grads_f32, cudaStream_t stream) {
    using bf = __nv_bfloat16;
    if (dtype == FDMLA_F32) return launch_bwd_t<float, float>(p, stream);
    if (dtype == FDMLA_BF16)
        return grads_f32 ? launch_bwd_t<bf, float>(p, stream) : launch_bwd_t<bf, bf>(p, stream);
    return FDMLA_ERR_INVALID;
}

// ---------------------------------------------------------------------------
// Weight gradient dW[d_in, d_out] = sum_rows X[row, :]^T G[row, :] in two
// deterministic stages: each block reduces a strided set of 32-row tiles into
// a partial [d_in*d_out] slab, then a second kernel sums the slabs in order.
// ---------------------------------------------------------------------------
constexpr int WG_U = 32;   // outputs per thread (256 threads -> 8192 outputs per grid.y slab)

template <typename T>
__global__ void __launch_bounds__(256)
wgrad_partial_kernel(const T *__restrict__ X, const float *__restrict__ G, float *__restrict__ part,
                     long long rows, int d_in, int d_out) {
    extern __shared__ __align__(16) float smem[];
    float *Xs = smem;                 // [32][d_in]
    float *Gs = Xs + 32 * d_in;       // [32][d_out]
    const int tid = threadIdx.x;
    const int n_out = d_in * d_out;
    const int base = blockIdx.y * (256 * WG_U);
    float acc[WG_U];
#pragma unroll
    for (int u = 0; u < WG_U; ++u) acc[u] = 0.f;
    for (long long r0 = (long long)blockIdx.x * 32; r0 < rows; r0 += (long long)gridDim.x * 32) {
        __syncthreads();
        for (int idx = tid; idx < 32 * d_in; idx += 256) {
            int r = idx / d_in;
            Xs[idx] = (r0 + r < rows) ? to_f32(X[(size_t)r0 * d_in + idx]) : 0.f;
        }
        for (int idx = tid; idx < 32 * d_out; idx += 256) {
            int r = idx / d_out;
            Gs[idx] = (r0 + r < rows) ? G[(size_t)r0 * d_out + idx] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < WG_U; ++u) {
            int o = base + tid + 256 * u;
            if (o < n_out) {
                int c = o / d_out, n = o - c * d_out;
                float a = acc[u];
                for (int r = 0; r < 32; ++r) a = fmaf(Xs[r * d_in + c], Gs[r * d_out + n], a);
                acc[u] = a;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < WG_U; ++u) {
        int o = base + tid + 256 * u;
        if (o < n_out) part[(size_t)blockIdx.x * n_out + o] = acc[u];
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
wgrad_reduce_kernel(const float *__restrict__ part, T *__restrict__ dW, int n_out, int n_part) {
    int o = blockIdx.x * 256 + threadIdx.x;
    if (o >= n_out) return;
    float acc = 0.f;
    for (int q = 0; q < n_part; ++q) acc += part[(size_t)q * n_out + o];
    dW[o] = from_f32<T>(acc);
}

int wgrad_num_partials(long long rows) {
    long long tiles = (rows + 31) / 32;
    long long n = 2 * kNumSMs;
    return (int)(tiles < n ? (tiles > 0 ? tiles : 1) : n);
}

int launch_wgrad(const void *X, const float *G, float *partials, void *dW, long long rows,
                 int d_in, int d_out, int dtype, cudaStream_t stream) {
    const int n_out = d_in * d_out;
    const int n_part = wgrad_num_partials(rows);
    size_t bytes = (size_t)32 * (d_in + d_out) * sizeof(float);
    if (bytes > (size_t)kMaxSmemPerBlock) return FDMLA_ERR_UNSUPPORTED;
    dim3 grid(n_part, (n_out + 256 * WG_U - 1) / (256 * WG_U));
    using bf = __nv_bfloat16;
    if (dtype == FDMLA_F32) {
        cudaFuncSetAttribute(wgrad_partial_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        wgrad_partial_kernel<float><<<grid, 256, bytes, stream>>>(static_cast<const float *>(X), G, partials, rows, d_in, d_out);
        wgrad_reduce_kernel<float><<<(n_out + 255) / 256, 256, 0, stream>>>(partials, static_cast<float *>(dW), n_out, n_part);
    } else if (dtype == FDMLA_BF16) {
        int rc = tensor_kernels_allowed() ? launch_wgrad_partial_tensor(X, G, partials, rows, d_in, d_out, n_part, stream)
                                          : FDMLA_ERR_UNSUPPORTED;
        if (rc != FDMLA_OK && rc != FDMLA_ERR_UNSUPPORTED) return rc;
        if (rc == FDMLA_ERR_UNSUPPORTED) {
            cudaFuncSetAttribute(wgrad_partial_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            wgrad_partial_kernel<bf><<<grid, 256, bytes, stream>>>(static_cast<const bf *>(X), G, partials, rows, d_in, d_out);
        }
        wgrad_reduce_kernel<bf><<<(n_out + 255) / 256, 256, 0, stream>>>(partials, static_cast<bf *>(dW), n_out, n_part);
    } else {
        return FDMLA_ERR_INVALID;
    }
    return check_launch();
}

}  // namespace fdmla
