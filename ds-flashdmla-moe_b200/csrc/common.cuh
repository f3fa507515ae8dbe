// Shared definitions for the Flash-DMLA kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/flashdmla.h"

namespace fdmla {

constexpr int kNumSMs = 148;            // B200: 2 dies x 74 SMs
constexpr int kMaxSmemPerBlock = 232448; // 227 KB opt-in shared memory per CTA

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Description of one forward/decode problem in the "row" form every forward
// kernel uses.  A KV group g owns R = heads_per_group * Sq query rows that all
// attend the same latent rows:
//   cache-latent: group = batch b,      R = H * Sq  (K_lat shared by the heads)
//   on-the-fly:   group = (b, h) pair,  R = Sq      (per-head projected latents)
//   decode:       group = sequence b,   R = H       (Sq = 1)
// Row r of a group is query i = r % Sq; it sees keys t with
//   kv_lo <= t < min(kv_hi, i + seqlen - Sq + 1 if causal else seqlen).
struct FwdProblem {
    const void *Q;            // [G, R, d_qk]
    const void *K;            // dense: [G, Skv, d_qk]; paged: pool [pages, page, d_qk]
    const void *V;            // dense: [G, Skv, ldv];  nullptr => V = K[..., :d_v]
    const int32_t *page_table; // [G, max_pages] or nullptr (dense)
    const int32_t *seqlens;    // [G] or nullptr (=> Skv)
    void *O;                  // [G, R, d_v] in dtype (final) - may be null when partial only
    float *m, *l;             // [G, R]
    float *O_part;            // [splits, G, R, d_v]
    float *m_part, *l_part;   // [splits, G, R]
    int G, R, Sq, Skv;
    int d_qk, d_v;
    int page_size, max_pages, num_pages;
    int num_splits;
    int kv_begin, kv_end;     // attended token window (kv_end < 0: unlimited)
    int causal;
    float scale;
    // Balanced decode schedule of the 2-CTA tensor kernel (0 = off): keys are handed out as contiguous
    // runs of 256-key tiles, at least quota_min per CTA pair; num_splits then counts the partial slabs.
    int balanced, quota_min;     // balanced: 0 no, 1 with a final output, 2 every piece (also of uncut sequences) a partial
    // Balanced schedule only: arrival counters [2 G], zero at launch.  When given, the CTA that finishes the last
    // piece of a cut sequence merges the pieces itself and no merge kernel is needed; nullptr = merge kernel.
    unsigned int *tickets;
};

// Token range [lo, hi) of split `s` for a group whose attended window is
// [w_lo, w_hi): contiguous pieces of whole `gran`-token blocks, the remainder
// spread over the first splits (the balanced rule of the reference's KV
// partitioning, csrc/attention/fa2_fwd_mpi.cu:47-53, applied to blocks).
__host__ __device__ __forceinline__ void split_window(int w_lo, int w_hi, int gran, int s,
                                                      int num_splits, int *lo, int *hi) {
    if (w_hi <= w_lo) { *lo = *hi = w_lo; return; }
    int first_blk = w_lo / gran;
    int last_blk = (w_hi + gran - 1) / gran;       // exclusive
    int nblk = last_blk - first_blk;
    int base = nblk / num_splits, rem = nblk % num_splits;
    int b0 = first_blk + s * base + (s < rem ? s : rem);
    int b1 = b0 + base + (s < rem ? 1 : 0);
    int a = b0 * gran, b = b1 * gran;
    *lo = a < w_lo ? w_lo : a;
    *hi = b > w_hi ? w_hi : b;
    if (*hi < *lo) *hi = *lo;
}

// Launchers implemented in the .cu files; all return a FDMLA_* status.
int launch_fwd_portable(const FwdProblem &p, int dtype, cudaStream_t stream);
int launch_fwd_tensor(const FwdProblem &p, int dtype, cudaStream_t stream);   // tcgen05
bool fwd_tensor_supported(const FwdProblem &p, int dtype);
int tensor_error_flag(int reset);        // device-side time-out / bad-page flag of the tcgen05 kernels
void tensor_prefer_single_cta(int on);   // keep MLA shapes on the 1-CTA kernel (A/B tests)
bool tensor_single_cta_preferred();
int launch_merge(const float *O_part, const float *m_part, const float *l_part, void *O,
                 float *m, float *l, long long rows, int d_v, int num_parts, int out_dtype,
                 cudaStream_t stream);
int launch_merge_strided(const float *O_part, const float *m_part, const float *l_part, void *O,
                         float *m, float *l, long long rows, int d_v, int num_parts, size_t part_stride_o,
                         size_t part_stride_ml, int out_dtype, cudaStream_t stream);
// 2-CTA tensor kernel: does it take this problem, and how many of its CTA pairs run at once on this device
bool fwd_tensor2_supported(const FwdProblem &p, int dtype);
int fwd_tensor2_resident_clusters();
int launch_project(const void *X, const void *W, void *Y, long long rows, int d_in, int d_out,
                   int w_transposed, int x_f32, int dtype, cudaStream_t stream);

struct BwdProblem {
    const void *Q;        // [G, R, d_qk], R = Hg*Sq rows sharing group g's keys
    const void *K;        // [G, Skv, d_qk]
    const void *V;        // [G, Skv, d_v] or nullptr (V = K[..., :d_v])
    const void *O, *dO;   // [G, R, d_v]
    const float *m, *l;   // [G, R]
    float *D;             // [G, R] scratch: rowsum(dO o O)
    void *dQ;             // [G, R, d_qk]  (dtype)
    void *dK;             // [G, Skv, d_qk] (fp32 or dtype, see dkv_f32)
    void *dV;             // [G, Skv, d_v]; unused when V aliases K (folded into dK)
    int G, R, Sq, Skv, d_qk, d_v, causal;
    float scale;
};

int launch_bwd_portable(const BwdProblem &p, int dtype, int grads_f32, cudaStream_t stream);
// D = rowsum(dO o O) alone (the first step of launch_bwd_portable)
int launch_bwd_delta(const BwdProblem &p, int dtype, cudaStream_t stream);
// tcgen05 backward of the attention core: bf16, 64-wide latents with a separate V, fp32 dK/dV
bool bwd_tensor_supported(const BwdProblem &p, int dtype, int grads_f32);
int launch_bwd_tensor(const BwdProblem &p, cudaStream_t stream);
int bwd_tensor_error_flag(int reset);
// batched bf16 GEMM on tcgen05 (csrc/tc_gemm.cu) and the RoPE tail of the absorbed query
// Causal hint for a GEMM of the attention backward: row m of an entry is query position (row0 + m) mod period and sees
// columns (mode 1: S, dP - tiles nobody sees are neither computed nor written) or reduction indices (mode 2: dQ = dS K)
// up to position + off.
struct GemmCausalHint { int mode, period, off; long long row0; };
int launch_gemm_batched(const void *A, const void *B, const void *B2, void *C, int batch, int M, int N, int K,
                        long long a_rows, long long lda, int a_brow, int a_bcol, long long b_rows, long long ldb,
                        int b_brow, int b_bcol, int b_k_major, long long ldc, long long c_brow, long long c_bcol,
                        int gated, const int32_t *row_offsets, cudaStream_t stream, float alpha = 1.f, int c_f32 = 0,
                        int accumulate = 0,
                        const GemmCausalHint *causal = nullptr);
// cache-latent backward as GEMMs on the tensor cores with the score matrices in a workspace (csrc/cl_bwd.cu)
bool bwd_cache_latent_tensor_supported(const BwdProblem &p, int dtype);
size_t bwd_cache_latent_tensor_workspace(int G, long long R, int Skv, int d_qk);
int launch_bwd_cache_latent_tensor(const BwdProblem &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int launch_rope_rows(const void *x, long long ldx, void *y, long long ldy, const int32_t *pos, long long rows,
                     int rows_per_pos, int d, float base, cudaStream_t stream);
int gemm_error_flag(int reset);
int exchange_error_flag(int reset);
size_t exchange_bytes(int world, long long rows, int d_v);
int launch_exchange_merge(const float *O_part, const float *m_part, const float *l_part, int num_parts, void *msg,
                          void *const *bufs, int world, int rank, long long rows, int d_v, void *O,
                          float *m, float *l, int out_dtype, int timeout_ms, cudaStream_t stream);
// tcgen05 projections / weight-gradient partials for widths (128 -> 64) and (64 -> 128 transposed); they return
// FDMLA_ERR_UNSUPPORTED for other shapes
int launch_project_tensor(const void *X, const void *W, void *Y, long long rows, int d_in, int d_out, int w_transposed,
                          int x_f32, cudaStream_t stream);
int launch_wgrad_partial_tensor(const void *X, const float *G, float *part, long long rows, int d_in, int d_out, int n_part,
                                cudaStream_t stream);
// false when the caller has forced the CUDA-core kernels (fdmla_set_backend)
bool tensor_kernels_allowed();
int wgrad_num_partials(long long rows);
int launch_wgrad(const void *X, const float *G, float *partials, void *dW, long long rows,
                 int d_in, int d_out, int dtype, cudaStream_t stream);

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FDMLA_OK : FDMLA_ERR_CUDA;
}

}  // namespace fdmla
