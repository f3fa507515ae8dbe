// Cache-latent DMLA backward on the tensor cores, unfused: the score matrices of a block of query rows go through a
// workspace and every matrix product is one launch of the batched tcgen05 GEMM (csrc/tc_gemm.cu).
//
// Per KV group g (a batch entry: its R = H * Sq query rows share the latent rows K [Skv, d_qk], V = K[:, :d_v]) and
// per chunk of RC query rows, with the formulas the reference intends in csrc/attention/fa2_bwd.cu (delta :198-216,
// dS = P (dP - delta) :234, dK :252-254, dV :259-272, dQ :293-309) and the softmax scale applied:
//   S   = Q K^T                     fp32 [RC, Skv]    GEMM (B K-major)
//   dP  = dO V^T                    fp32 [RC, Skv]    GEMM (B = the first d_v columns of K)
//   P   = exp(scale S - m) / l  (0 where masked),  dS = P o (dP - D)         one elementwise kernel, which writes
//         dS [RC, Skv] and the transposes dS^T, P^T [Skv, RC] in bf16
//   dQ  = scale dS K                bf16 [RC, d_qk]   GEMM (B MN-major)
//   dK += scale dS^T Q              fp32 [Skv, d_qk]  GEMM, accumulated over the chunks
//   dK[:, :d_v] += P^T dO                             GEMM (the value gradient folds into the latent's first columns)
// and dK is converted to the caller's dtype at the end of the group.  It computes the masked half of a causal problem
// too and moves 14 bytes per score through HBM - a fused kernel would not - but it runs the 2 x (3 d_qk + 2 d_v) FLOP
// per score on the tensor cores instead of the CUDA cores.  bf16, d_qk, d_v, Skv multiples of 64.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common.cuh"

namespace fdmla {
namespace clb {

constexpr long long kChunkBytes = 1ll << 31;      // bound on the score workspace of one chunk (14 bytes per score)
constexpr long long kChunkRowsMax = 131072;       // and on its rows (the elementwise kernel's grid: rows / 32 <= 65535)

__host__ __device__ inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

// rows of one chunk: a multiple of 128, at most what 2 GB of score workspace hold, at most the group's rows
static int chunk_rows(long long R, int Skv) {
    long long rc = kChunkBytes / ((long long)Skv * 14) / 128 * 128;
    if (rc < 128) rc = 128;
    if (rc > kChunkRowsMax) rc = kChunkRowsMax;
    const long long r_up = round_up(R, 128);
    return (int)(rc < r_up ? rc : r_up);
}

// The dK GEMMs have few output tiles (Skv / 128 x d_qk / 256) and a long reduction (the chunk's rows): they run as a
// batch of `ks` slices of the reduction, each into its own fp32 slab, so that the GPU is filled; the slabs are summed
// when the group is converted.
static int k_slices(int rc, int Skv, int d_qk) {
    const int tiles = ((Skv + 127) / 128) * ((d_qk + 255) / 256);
    int ks = 1;
    while (ks < 16 && tiles * ks < 296 && (rc / (2 * ks)) % 64 == 0 && rc / (2 * ks) >= 64) ks *= 2;
    return ks;
}

struct Layout { size_t D, dKacc, S, dP, dS, dST, PT, total; int rc, ks; };
static Layout layout(int G, long long R, int Skv, int d_qk) {
    Layout L{};
    L.rc = chunk_rows(R, Skv);
    L.ks = k_slices(L.rc, Skv, d_qk);
    auto al = [](size_t x) { return (x + 255) & ~size_t(255); };
    size_t off = 0;
    L.D = off; off += al((size_t)G * R * 4);
    L.dKacc = off; off += al((size_t)L.ks * Skv * d_qk * 4);
    L.S = off; off += al((size_t)L.rc * Skv * 4);
    L.dP = off; off += al((size_t)L.rc * Skv * 4);
    L.dS = off; off += al((size_t)L.rc * Skv * 2);
    L.dST = off; off += al((size_t)Skv * L.rc * 2);
    L.PT = off; off += al((size_t)Skv * L.rc * 2);
    L.total = off;
    return L;
}

// One 64 x 64 tile of scores per block of 256 threads.  Rows r0 .. of the chunk are rows row_base + r of the group.
// Pass 1: a thread takes four keys (one 16-byte vector of S and of dP) of four rows - all eight loads issued before the
// first use; vectors a causal row cannot see are not loaded at all - forms P and dS, stores dS as 8 bytes and drops both
// into shared memory transposed.  Pass 2: eight rows (16 bytes) of one key per thread to P^T and dS^T.
constexpr int SG_T = 64, SG_LD = SG_T + 8;       // tile edge; row pitch of the transposed tiles in bf16 (16-byte multiples)
__global__ void __launch_bounds__(256)
softmax_grad_kernel(const float *__restrict__ S, const float *__restrict__ dP, const float *__restrict__ m,
                    const float *__restrict__ l, const float *__restrict__ D, __nv_bfloat16 *__restrict__ dS,
                    __nv_bfloat16 *__restrict__ dST, __nv_bfloat16 *__restrict__ PT, int rc, int rows_valid, int Skv,
                    long long row_base, int Sq, int causal, float scale) {
    __shared__ __align__(16) __nv_bfloat16 tp[SG_T][SG_LD], tds[SG_T][SG_LD];      // [key][row]
    const int k0 = blockIdx.x * SG_T, r0 = blockIdx.y * SG_T;
    const int tid = threadIdx.x;
    const int kq = (tid & 15) * 4;                 // this thread's four keys inside the tile
    const float sl2 = scale * 1.4426950408889634f;
    const int off = Skv - Sq;                      // key j is visible to query position i iff j <= i + off
    float4 sv[4], dv[4];
    float mv[4], lv[4], Dv[4];
    int lim[4];                                    // last visible key of the row (-1: the row holds nothing)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + (tid >> 4) + 16 * i;
        lim[i] = -1;
        mv[i] = 0.f; lv[i] = 0.f; Dv[i] = 0.f;
        sv[i] = dv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows_valid) {
            const long long gr = row_base + r;
            lv[i] = l[gr];
            if (lv[i] > 0.f) lim[i] = causal ? (int)(gr % Sq) + off : Skv - 1;
            if (k0 + kq <= lim[i]) {
                mv[i] = m[gr]; Dv[i] = D[gr];
                const size_t idx = (size_t)r * Skv + k0 + kq;
                sv[i] = *reinterpret_cast<const float4 *>(S + idx);
                dv[i] = *reinterpret_cast<const float4 *>(dP + idx);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rr = (tid >> 4) + 16 * i, r = r0 + rr;
        const float s4[4] = {sv[i].x, sv[i].y, sv[i].z, sv[i].w}, d4[4] = {dv[i].x, dv[i].y, dv[i].z, dv[i].w};
        __nv_bfloat16 pb[4], db[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float pe = 0.f, de = 0.f;
            if (k0 + kq + e <= lim[i]) {
                pe = exp2f(fmaf(s4[e], sl2, -mv[i] * 1.4426950408889634f)) / lv[i];
                de = pe * (d4[e] - Dv[i]);
            }
            pb[e] = __float2bfloat16(pe);
            db[e] = __float2bfloat16(de);
            tp[kq + e][rr] = pb[e];
            tds[kq + e][rr] = db[e];
        }
        if (r < rc) {
            uint2 w;
            w.x = (uint32_t)__bfloat16_as_ushort(db[0]) | ((uint32_t)__bfloat16_as_ushort(db[1]) << 16);
            w.y = (uint32_t)__bfloat16_as_ushort(db[2]) | ((uint32_t)__bfloat16_as_ushort(db[3]) << 16);
            *reinterpret_cast<uint2 *>(dS + (size_t)r * Skv + k0 + kq) = w;
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int kk = (tid >> 3) + 32 * i, r8 = (tid & 7) * 8;
        if (r0 + r8 < rc) {                        // rc is a multiple of 128: a vector of eight rows is inside or outside
            const size_t o = (size_t)(k0 + kk) * rc + r0 + r8;
            *reinterpret_cast<uint4 *>(PT + o) = *reinterpret_cast<const uint4 *>(&tp[kk][r8]);
            *reinterpret_cast<uint4 *>(dST + o) = *reinterpret_cast<const uint4 *>(&tds[kk][r8]);
        }
    }
}

// dst = sum of the `slabs` fp32 slabs of n elements each, as bf16
__global__ void to_bf16_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, long long n, int slabs) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        float4 v = *reinterpret_cast<const float4 *>(src + i);
        for (int s2 = 1; s2 < slabs; ++s2) {
            const float4 u = *reinterpret_cast<const float4 *>(src + (size_t)s2 * n + i);
            v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
        }
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2 *>(dst + i) = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
    } else {
        for (long long j = i; j < n; ++j) {
            float v = src[j];
            for (int s2 = 1; s2 < slabs; ++s2) v += src[(size_t)s2 * n + j];
            dst[j] = __float2bfloat16(v);
        }
    }
}

}  // namespace clb

bool bwd_cache_latent_tensor_supported(const BwdProblem &p, int dtype) {
    if (dtype != FDMLA_BF16 || !tensor_kernels_allowed()) return false;
    if (p.V != nullptr || p.d_qk % 64 != 0 || p.d_v % 64 != 0 || p.Skv % 64 != 0 || p.d_v > p.d_qk) return false;
    if (p.G <= 0 || p.R <= 0 || p.Skv <= 0 || p.Sq <= 0) return false;
    if ((long long)p.G * p.R > 2147483647LL || (long long)p.G * p.Skv > 2147483647LL) return false;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p.Q) | reinterpret_cast<uintptr_t>(p.K) | reinterpret_cast<uintptr_t>(p.dO) |
                        reinterpret_cast<uintptr_t>(p.dQ) | reinterpret_cast<uintptr_t>(p.dK);
    return (a & 31) == 0;
}

size_t bwd_cache_latent_tensor_workspace(int G, long long R, int Skv, int d_qk) { return clb::layout(G, R, Skv, d_qk).total; }

int launch_bwd_cache_latent_tensor(const BwdProblem &p_in, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    using namespace clb;
    const Layout L = layout(p_in.G, p_in.R, p_in.Skv, p_in.d_qk);
    if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return FDMLA_ERR_WORKSPACE;
    char *ws = static_cast<char *>(workspace);
    BwdProblem p = p_in;
    p.D = reinterpret_cast<float *>(ws + L.D);
    int rc_status = launch_bwd_delta(p, FDMLA_BF16, stream);
    if (rc_status) return rc_status;
    float *dKacc = reinterpret_cast<float *>(ws + L.dKacc);
    float *S = reinterpret_cast<float *>(ws + L.S), *dP = reinterpret_cast<float *>(ws + L.dP);
    __nv_bfloat16 *dS = reinterpret_cast<__nv_bfloat16 *>(ws + L.dS), *dST = reinterpret_cast<__nv_bfloat16 *>(ws + L.dST),
                  *PT = reinterpret_cast<__nv_bfloat16 *>(ws + L.PT);
    const int Skv = p.Skv, dq = p.d_qk, dv = p.d_v, RC = L.rc;
    const __nv_bfloat16 *Q = static_cast<const __nv_bfloat16 *>(p.Q), *K = static_cast<const __nv_bfloat16 *>(p.K),
                        *dO = static_cast<const __nv_bfloat16 *>(p.dO);
    __nv_bfloat16 *dQ = static_cast<__nv_bfloat16 *>(p.dQ), *dK = static_cast<__nv_bfloat16 *>(p.dK);
    auto gemm = [&](const void *A, long long a_rows, long long lda, const void *B, long long b_rows, long long ldb, int k_major,
                    void *C, long long ldc, int M, int N, int Kd, float alpha, int c_f32, int acc,
                    const GemmCausalHint *hint = nullptr) {
        return launch_gemm_batched(A, B, nullptr, C, 1, M, N, Kd, a_rows, lda, 0, 0, b_rows, ldb, 0, 0, k_major, ldc, 0, 0, 0,
                                   nullptr, stream, alpha, c_f32, acc, hint);
    };
    for (int g = 0; g < p.G; ++g) {
        const __nv_bfloat16 *Kg = K + (size_t)g * Skv * dq;
        for (long long r0 = 0; r0 < p.R; r0 += RC) {
            const int rows = (int)((p.R - r0) < RC ? (p.R - r0) : RC);
            const long long grow = (long long)g * p.R + r0;
            const __nv_bfloat16 *Qc = Q + grow * dq, *dOc = dO + grow * dv;
            int rc;
            // S = Q K^T, dP = dO V^T (rows past the chunk's end read as zero: the tensor maps end there)
            // causal: score tiles that no row of the tile sees are neither computed nor written (the elementwise kernel
            // does not read them), and the reduction of dQ stops behind the last key a tile's rows see
            const GemmCausalHint skip{p.causal ? 1 : 0, p.Sq, Skv - p.Sq, grow}, limit{p.causal ? 2 : 0, p.Sq, Skv - p.Sq, grow};
            if ((rc = gemm(Qc, rows, dq, Kg, Skv, dq, 1, S, Skv, rows, Skv, dq, 1.f, 1, 0, &skip))) return rc;
            if ((rc = gemm(dOc, rows, dv, Kg, Skv, dq, 1, dP, Skv, rows, Skv, dv, 1.f, 1, 0, &skip))) return rc;
            softmax_grad_kernel<<<dim3(Skv / clb::SG_T, RC / clb::SG_T), 256, 0, stream>>>(
                S, dP, p.m, p.l, p.D, dS, dST, PT, RC, rows, Skv, grow, p.Sq, p.causal, p.scale);
            if ((rc = check_launch())) return rc;
            // dQ = scale dS K
            if ((rc = gemm(dS, rows, Skv, Kg, Skv, dq, 0, dQ + grow * dq, dq, rows, dq, Skv, p.scale, 0, 0, &limit))) return rc;
            // dK (+)= scale dS^T Q;  dK[:, :d_v] += P^T dO   (reduction over the chunk's rows, zero-padded to RC, in KS
            // slices that run as a batch: slice s reads columns s RC/KS .. of dS^T / P^T and the same rows of Q / dO and
            // accumulates into slab s)
            const int KS = L.ks, kslice = RC / KS;
            if ((rc = launch_gemm_batched(dST, Qc, nullptr, dKacc, KS, Skv, dq, kslice, Skv, RC, 0, kslice, rows, dq, kslice, 0, 0, dq,
                                          Skv, 0, 0, nullptr, stream, p.scale, 1, r0 > 0)))
                return rc;
            if ((rc = launch_gemm_batched(PT, dOc, nullptr, dKacc, KS, Skv, dv, kslice, Skv, RC, 0, kslice, rows, dv, kslice, 0, 0, dq,
                                          Skv, 0, 0, nullptr, stream, 1.f, 1, 1)))
                return rc;
        }
        const long long n = (long long)Skv * dq;
        to_bf16_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, stream>>>(dKacc, dK + (size_t)g * n, n, L.ks);
        const int rc = check_launch();
        if (rc) return rc;
    }
    return FDMLA_OK;
}

}  // namespace fdmla
