// extern "C" entry points of libflashdmla.so: argument checks, problem
// set-up and dispatch to the tcgen05 or the portable kernels.  Nothing here
// allocates or synchronises; every scratch buffer comes from the caller (the
// one exception: fdmla_exchange_alloc / _free, the set-up of an exchange buffer).
#include <cmath>
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace fdmla {

static std::atomic<int> g_backend{FDMLA_BACKEND_AUTO};
static thread_local const char *t_last_kernel = "none";

static inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
static inline size_t elem_size(int dtype) { return dtype == FDMLA_F32 ? 4 : 2; }
static inline bool dtype_ok(int dtype) { return dtype == FDMLA_F32 || dtype == FDMLA_BF16; }

bool tensor_kernels_allowed() { return g_backend.load() != FDMLA_BACKEND_PORTABLE; }

static int run_forward(const FwdProblem &p, int dtype, cudaStream_t stream) {
    const int backend = g_backend.load();
    const bool tc_ok = fwd_tensor_supported(p, dtype);
    if (backend == FDMLA_BACKEND_TENSOR && !tc_ok) return FDMLA_ERR_UNSUPPORTED;
    if (tc_ok && backend != FDMLA_BACKEND_PORTABLE) {
        t_last_kernel = "tcgen05";
        return launch_fwd_tensor(p, dtype, stream);
    }
    t_last_kernel = "portable";
    return launch_fwd_portable(p, dtype, stream);
}

// --- paged cache writer / gather -------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
cache_append_kernel(const T *__restrict__ rows, T *__restrict__ pool,
                    const int32_t *__restrict__ page_table, const int32_t *__restrict__ start_pos,
                    int n_tokens, int d, int page_size, int max_pages, int num_pages) {
    const int b = blockIdx.y, t = blockIdx.x;
    const int pos = start_pos[b] + t;
    const int lp = pos / page_size;
    if (pos < 0 || lp >= max_pages) return;
    const int pg = page_table[(size_t)b * max_pages + lp];
    if (pg < 0 || pg >= num_pages) return;
    const T *src = rows + ((size_t)b * n_tokens + t) * d;
    T *dst = pool + ((size_t)pg * page_size + (pos - lp * page_size)) * d;
    for (int k = threadIdx.x; k < d; k += blockDim.x) dst[k] = src[k];
}

template <typename T>
__global__ void __launch_bounds__(128)
cache_gather_kernel(const T *__restrict__ pool, const int32_t *__restrict__ page_table,
                    const int32_t *__restrict__ seqlens, T *__restrict__ out, int n_tokens, int d,
                    int page_size, int max_pages, int num_pages) {
    const int b = blockIdx.y, t = blockIdx.x;
    T *dst = out + ((size_t)b * n_tokens + t) * d;
    const int lp = t / page_size;
    int pg = -1;
    if (t < seqlens[b] && lp < max_pages) pg = page_table[(size_t)b * max_pages + lp];
    if (pg < 0 || pg >= num_pages) {
        for (int k = threadIdx.x; k < d; k += blockDim.x) dst[k] = from_f32<T>(0.f);
        return;
    }
    const T *src = pool + ((size_t)pg * page_size + (t - lp * page_size)) * d;
    for (int k = threadIdx.x; k < d; k += blockDim.x) dst[k] = src[k];
}

// CTA pairs the 2-CTA tensor kernel keeps resident on the current device (74 on a B200); the constant when there
// is no device to ask.
static int pair_units() {
    const int n = fwd_tensor2_resident_clusters();
    return n > 0 ? n : kNumSMs / 2;
}

static double equal_split_cost(long long items, int tiles, int s, int units) {
    const long long waves = (items * s + units - 1) / units;
    double cost = (double)waves * ((double)tiles / s + 1.5);
    if (s > 1) cost += 0.75 + 0.02 * s * (double)waves;   // merge launch + partial traffic
    return cost;
}

// How a decode call with `slabs` partial slabs runs on the 2-CTA tensor kernel when a final result is wanted.
// Costs are in tile times (a 256-key tile of one CTA pair), for sequences of the maximum length.
//   EQUAL               every sequence in `slabs` equal pieces, merge kernel
//   BALANCED_MERGE      the tiles of all sequences in equal contiguous runs, a sequence cut into at most `slabs`
//                       pieces, merge kernel over the cut rows (launch + partial traffic: about 7 tile times)
//   BALANCED_IN_KERNEL  the same runs with at most min(slabs - 1, kMaxInKernelPieces) pieces per sequence, merged by
//                       the CTA pair that finishes a sequence's last piece; the last slab holds the arrival counters
//                       (about 6 tile times for the partial rows, the counters and that merge)
constexpr int kMaxInKernelPieces = 4;
struct DecodePlan { enum Mode { EQUAL, BALANCED_MERGE, BALANCED_IN_KERNEL } mode; int quota_min; double cost; };

static DecodePlan plan_decode(int B, int nt_max, int slabs, int units) {
    DecodePlan best{DecodePlan::EQUAL, 0, equal_split_cost(B, nt_max, slabs, units)};
    if (slabs < 2 || nt_max < 1) return best;
    const long long run = ((long long)B * nt_max + units - 1) / units;
    {   // pieces <= floor((nt - 1) / q) + 2 <= slabs  <=  q >= ceil(nt / (slabs - 1))
        const int qmin = (nt_max + slabs - 2) / (slabs - 1);
        const double cost = (double)(run > qmin ? run : qmin) + 1.5 + 7.0;
        if (cost < best.cost) best = DecodePlan{DecodePlan::BALANCED_MERGE, qmin, cost};
    }
    if (slabs >= 3) {
        const int pieces = slabs - 1 < kMaxInKernelPieces ? slabs - 1 : kMaxInKernelPieces;
        const int qmin = (nt_max + pieces - 2) / (pieces - 1);
        // measured at B = 128 x 4096 keys: a pair that handles two cut sequences pays about six tile times for the
        // fp32 partial rows it writes, the arrival counters and the merge of the sequence it finishes last
        const double cost = (double)(run > qmin ? run : qmin) + 1.5 + 6.0;
        if (cost < best.cost) best = DecodePlan{DecodePlan::BALANCED_IN_KERNEL, qmin, cost};
    }
    return best;
}

}  // namespace fdmla

using namespace fdmla;

extern "C" {

int fdmla_version(void) { return 100; }

const char *fdmla_status_string(int status) {
    switch (status) {
        case FDMLA_OK: return "ok";
        case FDMLA_ERR_INVALID: return "invalid argument";
        case FDMLA_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case FDMLA_ERR_CUDA: return "CUDA error";
        case FDMLA_ERR_WORKSPACE: return "workspace missing or too small";
        case FDMLA_ERR_SCRATCH_LIMIT: return "problem exceeds the built-in scratch of the no-allocation entry point";
        default: return "unknown status";
    }
}

int fdmla_set_backend(int backend) {
    if (backend < FDMLA_BACKEND_AUTO || backend > FDMLA_BACKEND_TENSOR) return FDMLA_ERR_INVALID;
    g_backend.store(backend);
    return FDMLA_OK;
}
int fdmla_get_backend(void) { return g_backend.load(); }
int fdmla_set_single_cta(int on) { tensor_prefer_single_cta(on != 0); return FDMLA_OK; }
const char *fdmla_last_kernel(void) { return t_last_kernel; }
int fdmla_device_error_flag(int reset) {
    const int fwd = tensor_error_flag(reset), bwd = bwd_tensor_error_flag(reset), gemm = gemm_error_flag(reset),
              xch = exchange_error_flag(reset);
    return fwd ? fwd : (bwd ? bwd : (gemm ? gemm : xch));
}

size_t fdmla_exchange_bytes(int world, long long rows, int d_v) { return exchange_bytes(world, rows, d_v); }

int fdmla_exchange_alloc(size_t bytes, void **buf, void *ipc_handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the header promises a 64-byte handle");
    if (!buf || !ipc_handle || bytes == 0) return FDMLA_ERR_INVALID;
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return FDMLA_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return FDMLA_ERR_CUDA;
    }
    memcpy(ipc_handle, &h, sizeof(h));
    *buf = p;
    return FDMLA_OK;
}

int fdmla_exchange_open(const void *ipc_handle, void **peer_buf) {
    if (!ipc_handle || !peer_buf) return FDMLA_ERR_INVALID;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    void *p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return FDMLA_ERR_CUDA; }
    *peer_buf = p;
    return FDMLA_OK;
}

int fdmla_exchange_close(void *peer_buf) {
    if (!peer_buf) return FDMLA_OK;
    if (cudaIpcCloseMemHandle(peer_buf) != cudaSuccess) { cudaGetLastError(); return FDMLA_ERR_CUDA; }
    return FDMLA_OK;
}

int fdmla_exchange_free(void *buf) {
    if (!buf) return FDMLA_OK;
    if (cudaFree(buf) != cudaSuccess) { cudaGetLastError(); return FDMLA_ERR_CUDA; }
    return FDMLA_OK;
}

int fdmla_exchange_merge(const float *msg, void *const *bufs, int world, int rank, long long rows, int d_v, void *O,
                         float *m, float *l, int out_dtype, int timeout_ms, void *stream) {
    const int rc = launch_exchange_merge(nullptr, nullptr, nullptr, 0, const_cast<float *>(msg), bufs, world, rank, rows, d_v,
                                         O, m, l, out_dtype, timeout_ms, static_cast<cudaStream_t>(stream));
    if (rc == FDMLA_OK && rows > 0) t_last_kernel = "exchange_merge_kernel";
    return rc;
}

int fdmla_exchange_merge_parts(const float *O_part, const float *m_part, const float *l_part, int num_parts, float *msg,
                               void *const *bufs, int world, int rank, long long rows, int d_v, void *O, float *m,
                               float *l, int out_dtype, int timeout_ms, void *stream) {
    if (num_parts < 1) return FDMLA_ERR_INVALID;
    const int rc = launch_exchange_merge(O_part, m_part, l_part, num_parts, msg, bufs, world, rank, rows, d_v, O, m, l,
                                         out_dtype, timeout_ms, static_cast<cudaStream_t>(stream));
    if (rc == FDMLA_OK && rows > 0) t_last_kernel = "exchange_merge_kernel";
    return rc;
}

int fdmla_fwd_cache_latent(const void *Q, const void *K_lat, void *O, float *m, float *l, int B,
                           int H, int Sq, int Skv, int d_qk, int d_v, float scale, int causal,
                           int dtype, void *stream) {
    if (!dtype_ok(dtype)) return FDMLA_ERR_INVALID;
    if (B < 0 || H < 0 || Sq < 0 || Skv < 0 || d_qk <= 0 || d_v <= 0 || d_v > d_qk) return FDMLA_ERR_INVALID;
    if (B == 0 || H == 0 || Sq == 0) return FDMLA_OK;
    if (!Q || !O || !m || !l || (!K_lat && Skv > 0)) return FDMLA_ERR_INVALID;
    if ((long long)H * Sq > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    FwdProblem p{};
    p.Q = Q; p.K = K_lat; p.V = nullptr; p.page_table = nullptr; p.seqlens = nullptr;
    p.O = O; p.m = m; p.l = l;
    p.G = B; p.R = H * Sq; p.Sq = Sq; p.Skv = Skv; p.d_qk = d_qk; p.d_v = d_v;
    p.page_size = 0; p.max_pages = 0; p.num_pages = 0; p.num_splits = 1;
    p.kv_begin = 0; p.kv_end = -1; p.causal = causal ? 1 : 0; p.scale = scale;
    return run_forward(p, dtype, static_cast<cudaStream_t>(stream));
}

size_t fdmla_fwd_on_the_fly_workspace_bytes(int B, int H, int Skv, int d_lat, int dtype) {
    if (B <= 0 || H <= 0 || Skv <= 0 || d_lat <= 0 || !dtype_ok(dtype)) return 0;
    return 2 * align256((size_t)B * H * Skv * d_lat * elem_size(dtype));
}

int fdmla_fwd_on_the_fly(const void *Q, const void *K, const void *V, const void *WK,
                         const void *WV, void *O, float *m, float *l, void *workspace,
                         size_t workspace_bytes, int B, int H, int Sq, int Skv, int d_model,
                         int d_lat, float scale, int causal, int dtype, void *stream) {
    if (!dtype_ok(dtype)) return FDMLA_ERR_INVALID;
    if (B < 0 || H < 0 || Sq < 0 || Skv < 0 || d_model <= 0 || d_lat <= 0) return FDMLA_ERR_INVALID;
    if (B == 0 || H == 0 || Sq == 0) return FDMLA_OK;
    if (!Q || !O || !m || !l || !WK || !WV) return FDMLA_ERR_INVALID;
    if (Skv > 0 && (!K || !V)) return FDMLA_ERR_INVALID;
    const size_t need = fdmla_fwd_on_the_fly_workspace_bytes(B, H, Skv, d_lat, dtype);
    if (need > 0 && (!workspace || workspace_bytes < need)) return FDMLA_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return FDMLA_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    void *K_lat = ws;
    void *V_lat = ws + need / 2;
    const long long nkv = (long long)B * H * Skv;
    int rc = launch_project(K, WK, K_lat, nkv, d_model, d_lat, 0, 0, dtype, st);
    if (rc) return rc;
    rc = launch_project(V, WV, V_lat, nkv, d_model, d_lat, 0, 0, dtype, st);
    if (rc) return rc;
    FwdProblem p{};
    p.Q = Q; p.K = K_lat; p.V = V_lat; p.O = O; p.m = m; p.l = l;
    p.G = B * H; p.R = Sq; p.Sq = Sq; p.Skv = Skv; p.d_qk = d_lat; p.d_v = d_lat;
    p.num_splits = 1; p.kv_begin = 0; p.kv_end = -1; p.causal = causal ? 1 : 0; p.scale = scale;
    if (p.G > 65535) return FDMLA_ERR_UNSUPPORTED;
    return run_forward(p, dtype, st);
}

int fdmla_decode_suggest_splits(int B, int H, int max_seqlen, int d_qk, int d_v, int page_size,
                                int dtype) {
    if (B <= 0 || H <= 0 || max_seqlen <= 0 || page_size <= 0) return 1;
    // Cost model in units of one key tile of one work item.  The tcgen05 kernels run one
    // work item (128 rows x one split) per cluster of two CTAs in 256-key tiles, the other
    // kernels one 128-row item per CTA in 32-key tiles; each item pays a fixed cost of
    // about 1.5 tiles (Q load, pipeline fill, epilogue) and every split beyond the first
    // adds partial results that have to be written, read back and merged.
    const bool mla = (dtype == FDMLA_BF16 && d_qk == 576 && d_v == 512 && page_size % 64 == 0);
    const int tile = mla ? 256 : 32;
    const int units = mla ? pair_units() : kNumSMs;
    const long long items = (long long)B * ((H + 127) / 128) * ((mla || d_v <= 256) ? 1 : 2);
    const int tiles = (max_seqlen + tile - 1) / tile;
    const int pages = (max_seqlen + page_size - 1) / page_size;
    int best = 1;
    double best_cost = 1e30;
    const int s_max = tiles < pages ? tiles : pages;      // never less than one tile per split
    for (int s = 1; s <= 64 && s <= s_max; ++s) {
        const double cost = equal_split_cost(items, tiles, s, units);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    if (mla && H <= 128 && H >= 2 && tiles >= 1) {
        // Balanced schedule of the 2-CTA kernel (see DecodePlan): first with the merge inside the attention kernel,
        // which wants one slab more than the pieces a sequence may be cut into ...
        for (int pieces = 2; pieces <= kMaxInKernelPieces; ++pieces) {
            const DecodePlan pl = plan_decode(B, tiles, pieces + 1, units);
            if (pl.mode == DecodePlan::BALANCED_IN_KERNEL && pl.cost < best_cost - 1e-9) { best_cost = pl.cost; best = pieces + 1; }
        }
        // ... then with the merge kernel, for few long sequences that have to be cut many times: twice the pieces a
        // full-length sequence needs, since ragged batches have shorter runs than B x max and cut more often
        const double run = std::ceil((double)B * tiles / units);
        int slabs = 2 * (int)std::ceil(tiles / run) + 1;
        slabs = slabs < kMaxInKernelPieces + 2 ? kMaxInKernelPieces + 2 : (slabs > 64 ? 64 : slabs);
        const DecodePlan pl = plan_decode(B, tiles, slabs, units);
        if (pl.mode != DecodePlan::EQUAL && pl.cost < best_cost - 1e-9) { best_cost = pl.cost; best = slabs; }
    }
    return best;
}

int fdmla_decode_plan(int B, int H, int d_qk, int d_v, int page_size, int max_pages, int num_splits, int dtype,
                      int *quota_min, int *units) {
    if (quota_min) *quota_min = 0;
    if (units) *units = 0;
    if (B <= 0 || H <= 0 || page_size <= 0 || max_pages <= 0 || num_splits < 1) return FDMLA_ERR_INVALID;
    const bool mla = dtype == FDMLA_BF16 && d_qk == 576 && d_v == 512 && page_size % 64 == 0;
    if (!mla || num_splits < 2 || H > 128 || H < 2 || g_backend.load() == FDMLA_BACKEND_PORTABLE ||
        tensor_single_cta_preferred())
        return 0;
    const int nt_max = (int)(((long long)max_pages * page_size + 255) / 256);
    const int u = pair_units();
    const DecodePlan pl = plan_decode(B, nt_max, num_splits, u);
    if (units) *units = u;
    if (quota_min) *quota_min = pl.quota_min;
    return (int)pl.mode;
}

int fdmla_decode_paged(const void *Q, const void *kv_pool, const int32_t *page_table,
                       const int32_t *seqlens, void *O, float *m, float *l, float *O_part,
                       float *m_part, float *l_part, int B, int H, int d_qk, int d_v,
                       int page_size, int max_pages, int num_pages, int num_splits, int kv_begin,
                       int kv_end, float scale, int dtype, void *stream) {
    if (!dtype_ok(dtype)) return FDMLA_ERR_INVALID;
    if (B < 0 || H < 0 || d_qk <= 0 || d_v <= 0 || d_v > d_qk || page_size <= 0 || max_pages < 0 ||
        num_pages < 0 || num_splits < 1)
        return FDMLA_ERR_INVALID;
    if (B == 0 || H == 0) return FDMLA_OK;
    if (!Q || !kv_pool || !page_table || !seqlens) return FDMLA_ERR_INVALID;
    const bool partial_only = (O == nullptr);
    if (!partial_only && (!m || !l)) return FDMLA_ERR_INVALID;
    if ((num_splits > 1 || partial_only) && (!O_part || !m_part || !l_part)) return FDMLA_ERR_WORKSPACE;
    if (B > 65535) return FDMLA_ERR_UNSUPPORTED;
    if ((long long)max_pages * page_size > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdProblem p{};
    p.Q = Q; p.K = kv_pool; p.V = nullptr; p.page_table = page_table; p.seqlens = seqlens;
    p.O = (num_splits == 1) ? O : nullptr; p.m = m; p.l = l;
    p.O_part = O_part; p.m_part = m_part; p.l_part = l_part;
    p.G = B; p.R = H; p.Sq = 1; p.Skv = max_pages * page_size; p.d_qk = d_qk; p.d_v = d_v;
    p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages;
    p.num_splits = num_splits; p.kv_begin = kv_begin; p.kv_end = kv_end; p.causal = 0; p.scale = scale;
    bool merge_launch = num_splits > 1 && !partial_only;
    if (!partial_only && num_splits >= 2 && kv_begin <= 0 && kv_end < 0 && H <= 128 && H >= 2 &&
        g_backend.load() != FDMLA_BACKEND_PORTABLE && !tensor_single_cta_preferred() && fwd_tensor2_supported(p, dtype)) {
        // A final result is wanted and there are spare slabs: the 2-CTA tensor kernel may hand out the
        // keys as balanced runs of tiles instead of num_splits equal pieces of every sequence.  It writes
        // uncut sequences straight to O, so it needs O.
        const int nt_max = (int)(((long long)max_pages * page_size + 255) / 256);
        const DecodePlan pl = plan_decode(B, nt_max, num_splits, pair_units());
        if (pl.mode != DecodePlan::EQUAL) {
            p.balanced = 1;
            p.quota_min = pl.quota_min;
            p.O = O;
        }
        if (pl.mode == DecodePlan::BALANCED_IN_KERNEL) {
            // the arrival counters live in the last slab of l_part (no piece is ever written there: a sequence is cut
            // into num_splits - 1 pieces at most) and have to start at zero
            p.tickets = reinterpret_cast<unsigned int *>(l_part + (size_t)(num_splits - 1) * B * H);
            if (cudaMemsetAsync(p.tickets, 0, sizeof(unsigned int) * 2 * (size_t)B, st) != cudaSuccess) return FDMLA_ERR_CUDA;
            merge_launch = false;
        }
    }
    int rc = run_forward(p, dtype, st);
    if (rc) return rc;
    if (merge_launch)
        rc = launch_merge(O_part, m_part, l_part, O, m, l, (long long)B * H, d_v, num_splits, dtype, st);
    return rc;
}

int fdmla_decode_paged_partial(const void *Q, const void *kv_pool, const int32_t *page_table, const int32_t *seqlens,
                               float *O_out, float *m_out, float *l_out, float *O_part, float *m_part, float *l_part,
                               int B, int H, int d_qk, int d_v, int page_size, int max_pages, int num_pages,
                               int num_splits, float scale, int dtype, void *stream) {
    if (!dtype_ok(dtype)) return FDMLA_ERR_INVALID;
    if (B < 0 || H < 0 || d_qk <= 0 || d_v <= 0 || d_v > d_qk || page_size <= 0 || max_pages < 0 || num_pages < 0 ||
        num_splits < 1)
        return FDMLA_ERR_INVALID;
    if (B == 0 || H == 0) return FDMLA_OK;
    if (!Q || !kv_pool || !page_table || !seqlens) return FDMLA_ERR_INVALID;
    const bool pieces_only = !O_out && !m_out && !l_out && num_splits > 1;      // the caller merges the pieces itself
    if (!pieces_only && (!O_out || !m_out || !l_out)) return FDMLA_ERR_INVALID;
    if (num_splits > 1 && (!O_part || !m_part || !l_part)) return FDMLA_ERR_WORKSPACE;
    if (B > 65535 || (long long)max_pages * page_size > 2147483647LL) return FDMLA_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdProblem p{};
    p.Q = Q; p.K = kv_pool; p.V = nullptr; p.page_table = page_table; p.seqlens = seqlens;
    p.O = nullptr; p.m = nullptr; p.l = nullptr;
    p.G = B; p.R = H; p.Sq = 1; p.Skv = max_pages * page_size; p.d_qk = d_qk; p.d_v = d_v;
    p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages;
    p.num_splits = num_splits; p.kv_begin = 0; p.kv_end = -1; p.causal = 0; p.scale = scale;
    if (num_splits == 1) {        // one piece per sequence: the attention kernel writes the result itself
        p.O_part = O_out; p.m_part = m_out; p.l_part = l_out;
        return run_forward(p, dtype, st);
    }
    p.O_part = O_part; p.m_part = m_part; p.l_part = l_part;
    if (H <= 128 && H >= 2 && g_backend.load() != FDMLA_BACKEND_PORTABLE && !tensor_single_cta_preferred() &&
        fwd_tensor2_supported(p, dtype)) {
        // balanced runs of tiles, every piece a partial; a sequence is cut into at most num_splits pieces
        const int nt_max = (int)(((long long)max_pages * page_size + 255) / 256);
        p.balanced = 2;
        p.quota_min = (nt_max + num_splits - 2) / (num_splits - 1);
        if (p.quota_min < 1) p.quota_min = 1;
    }
    const int rc = run_forward(p, dtype, st);
    if (rc || pieces_only) return rc;
    return launch_merge(O_part, m_part, l_part, O_out, m_out, l_out, (long long)B * H, d_v, num_splits, FDMLA_F32, st);
}

int fdmla_gemm_batched(const void *A, const void *B, const void *B2, void *C, int batch, int M, int N, int K,
                       long long a_rows, long long lda, int a_brow, int a_bcol, long long b_rows, long long ldb,
                       int b_brow, int b_bcol, int b_k_major, long long ldc, long long c_brow, long long c_bcol,
                       int gated, void *stream) {
    if (batch < 0 || M < 0 || N < 0 || K < 0 || lda <= 0 || ldb <= 0 || ldc <= 0 || a_rows <= 0 || b_rows <= 0 ||
        a_brow < 0 || a_bcol < 0 || b_brow < 0 || b_bcol < 0 || c_brow < 0 || c_bcol < 0)
        return FDMLA_ERR_INVALID;
    if (batch == 0 || M == 0 || N == 0) return FDMLA_OK;
    if (!A || !B || !C || (gated && !B2) || K == 0) return FDMLA_ERR_INVALID;
    if (!tensor_kernels_allowed()) return FDMLA_ERR_UNSUPPORTED;
    // every window must lie inside its tensor (a copy that starts outside would read another tensor's rows as zeros
    // silently; a store outside would corrupt memory)
    if ((long long)(batch - 1) * a_brow + M > a_rows || (long long)(batch - 1) * a_bcol + K > lda) return FDMLA_ERR_INVALID;
    const long long b_need_rows = (long long)(batch - 1) * b_brow + (b_k_major ? N : K);
    const long long b_need_cols = (long long)(batch - 1) * b_bcol + (b_k_major ? K : N);
    if (b_need_rows > b_rows || b_need_cols > ldb) return FDMLA_ERR_INVALID;
    if ((batch - 1) * c_bcol + N > ldc) return FDMLA_ERR_INVALID;
    t_last_kernel = "tcgen05";
    return launch_gemm_batched(A, B, B2, C, batch, M, N, K, a_rows, lda, a_brow, a_bcol, b_rows, ldb, b_brow, b_bcol,
                               b_k_major, ldc, c_brow, c_bcol, gated, nullptr, static_cast<cudaStream_t>(stream));
}

int fdmla_gemm_grouped(const void *A, const void *B, const void *B2, void *C, const int32_t *row_offsets, int groups,
                       int total_rows, int N, int K, long long lda, long long b_rows, long long ldb, int b_brow,
                       int b_k_major, long long ldc, int gated, void *stream) {
    if (groups < 0 || total_rows < 0 || N < 0 || K < 0 || lda <= 0 || ldb <= 0 || ldc <= 0 || b_rows <= 0 || b_brow < 0)
        return FDMLA_ERR_INVALID;
    if (groups == 0 || total_rows == 0 || N == 0) return FDMLA_OK;
    if (!A || !B || !C || !row_offsets || (gated && !B2) || K == 0) return FDMLA_ERR_INVALID;
    if (!tensor_kernels_allowed()) return FDMLA_ERR_UNSUPPORTED;
    if (K > lda || N > ldc) return FDMLA_ERR_INVALID;
    const long long b_need_rows = (long long)(groups - 1) * b_brow + (b_k_major ? N : K);
    if (b_need_rows > b_rows || (b_k_major ? K : N) > ldb) return FDMLA_ERR_INVALID;
    t_last_kernel = "tcgen05";
    return launch_gemm_batched(A, B, B2, C, groups, total_rows, N, K, total_rows, lda, 0, 0, b_rows, ldb, b_brow, 0, b_k_major,
                               ldc, 0, 0, gated, row_offsets, static_cast<cudaStream_t>(stream));
}

int fdmla_rope_rows(const void *x, long long ldx, void *y, long long ldy, const int32_t *pos, long long rows,
                    int rows_per_pos, int d, float base, void *stream) {
    if (rows < 0) return FDMLA_ERR_INVALID;
    if (rows == 0) return FDMLA_OK;
    if (!x || !y || !pos) return FDMLA_ERR_INVALID;
    return launch_rope_rows(x, ldx, y, ldy, pos, rows, rows_per_pos, d, base, static_cast<cudaStream_t>(stream));
}

int fdmla_merge_lse(const float *O_part, const float *m_part, const float *l_part, void *O,
                    float *m, float *l, long long rows, int d_v, int num_parts, int out_dtype,
                    void *stream) {
    if (!dtype_ok(out_dtype) || rows < 0 || d_v <= 0 || num_parts < 1) return FDMLA_ERR_INVALID;
    if (rows == 0) return FDMLA_OK;
    if (!O_part || !m_part || !l_part || !O || !m || !l) return FDMLA_ERR_INVALID;
    return launch_merge(O_part, m_part, l_part, O, m, l, rows, d_v, num_parts, out_dtype,
                        static_cast<cudaStream_t>(stream));
}

int fdmla_merge_lse_strided(const float *O_part, const float *m_part, const float *l_part, void *O,
                            float *m, float *l, long long rows, int d_v, int num_parts,
                            long long part_stride_o, long long part_stride_ml, int out_dtype, void *stream) {
    if (!dtype_ok(out_dtype) || rows < 0 || d_v <= 0 || num_parts < 1) return FDMLA_ERR_INVALID;
    if (part_stride_o < rows * d_v || part_stride_ml < rows) return FDMLA_ERR_INVALID;
    if (rows == 0) return FDMLA_OK;
    if (!O_part || !m_part || !l_part || !O || !m || !l) return FDMLA_ERR_INVALID;
    return launch_merge_strided(O_part, m_part, l_part, O, m, l, rows, d_v, num_parts, (size_t)part_stride_o,
                                (size_t)part_stride_ml, out_dtype, static_cast<cudaStream_t>(stream));
}

// workspace of the on-the-fly backward:
//   K_lat, V_lat (dtype) | dK_lat, dV_lat (fp32) | D (fp32) | wgrad partial slabs (fp32)
struct BwdOtfLayout { size_t klat, vlat, dklat, dvlat, D, part, total; };
static BwdOtfLayout bwd_otf_layout(int B, int H, int Sq, int Skv, int d_model, int d_lat, int dtype) {
    BwdOtfLayout L{};
    const size_t nkv = (size_t)B * H * Skv, nq = (size_t)B * H * Sq;
    size_t off = 0;
    L.klat = off; off += align256(nkv * d_lat * elem_size(dtype));
    L.vlat = off; off += align256(nkv * d_lat * elem_size(dtype));
    L.dklat = off; off += align256(nkv * d_lat * 4);
    L.dvlat = off; off += align256(nkv * d_lat * 4);
    L.D = off; off += align256(nq * 4);
    L.part = off; off += align256((size_t)wgrad_num_partials((long long)nkv) * d_model * d_lat * 4);
    L.total = off;
    return L;
}

size_t fdmla_bwd_on_the_fly_workspace_bytes(int B, int H, int Sq, int Skv, int d_model, int d_lat,
                                            int dtype) {
    if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || d_model <= 0 || d_lat <= 0 || !dtype_ok(dtype)) return 0;
    return bwd_otf_layout(B, H, Sq, Skv, d_model, d_lat, dtype).total;
}

int fdmla_bwd_on_the_fly(const void *Q, const void *K, const void *V, const void *WK,
                         const void *WV, const void *O, const float *m, const float *l,
                         const void *dO, void *dQ, void *dK, void *dV, void *dWK, void *dWV,
                         void *workspace, size_t workspace_bytes, int B, int H, int Sq, int Skv,
                         int d_model, int d_lat, float scale, int causal, int dtype, void *stream) {
    if (!dtype_ok(dtype)) return FDMLA_ERR_INVALID;
    if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || d_model <= 0 || d_lat <= 0) return FDMLA_ERR_INVALID;
    if (!Q || !K || !V || !WK || !WV || !O || !m || !l || !dO || !dQ || !dK || !dV || !dWK || !dWV)
        return FDMLA_ERR_INVALID;
    const BwdOtfLayout L = bwd_otf_layout(B, H, Sq, Skv, d_model, d_lat, dtype);
    if (!workspace || workspace_bytes < L.total) return FDMLA_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return FDMLA_ERR_INVALID;
    if ((long long)B * H > 65535) return FDMLA_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    void *K_lat = ws + L.klat, *V_lat = ws + L.vlat;
    float *dK_lat = reinterpret_cast<float *>(ws + L.dklat);
    float *dV_lat = reinterpret_cast<float *>(ws + L.dvlat);
    const long long nkv = (long long)B * H * Skv;
    int rc = launch_project(K, WK, K_lat, nkv, d_model, d_lat, 0, 0, dtype, st);
    if (rc) return rc;
    rc = launch_project(V, WV, V_lat, nkv, d_model, d_lat, 0, 0, dtype, st);
    if (rc) return rc;
    BwdProblem p{};
    p.Q = Q; p.K = K_lat; p.V = V_lat; p.O = O; p.dO = dO; p.m = m; p.l = l;
    p.D = reinterpret_cast<float *>(ws + L.D);
    p.dQ = dQ; p.dK = dK_lat; p.dV = dV_lat;
    p.G = B * H; p.R = Sq; p.Sq = Sq; p.Skv = Skv; p.d_qk = d_lat; p.d_v = d_lat;
    p.causal = causal ? 1 : 0; p.scale = scale;
    const int backend = g_backend.load();
    const bool tc_ok = bwd_tensor_supported(p, dtype, 1);
    if (backend == FDMLA_BACKEND_TENSOR && !tc_ok) return FDMLA_ERR_UNSUPPORTED;
    if (tc_ok && backend != FDMLA_BACKEND_PORTABLE) {
        t_last_kernel = "tcgen05";
        rc = launch_bwd_delta(p, dtype, st);
        if (rc) return rc;
        rc = launch_bwd_tensor(p, st);
    } else {
        t_last_kernel = "portable";
        rc = launch_bwd_portable(p, dtype, /*grads_f32=*/1, st);
    }
    if (rc) return rc;
    // dK = dK_lat WK^T, dV = dV_lat WV^T
    rc = launch_project(dK_lat, WK, dK, nkv, d_lat, d_model, 1, 1, dtype, st);
    if (rc) return rc;
    rc = launch_project(dV_lat, WV, dV, nkv, d_lat, d_model, 1, 1, dtype, st);
    if (rc) return rc;
    // dWK = sum K^T dK_lat, dWV = sum V^T dV_lat
    float *part = reinterpret_cast<float *>(ws + L.part);
    rc = launch_wgrad(K, dK_lat, part, dWK, nkv, d_model, d_lat, dtype, st);
    if (rc) return rc;
    return launch_wgrad(V, dV_lat, part, dWV, nkv, d_model, d_lat, dtype, st);
}

size_t fdmla_bwd_cache_latent_workspace_bytes(int B, int H, int Sq, int Skv, int d_qk, int d_v,
                                              int dtype) {
    if (B <= 0 || H <= 0 || Sq <= 0 || !dtype_ok(dtype)) return 0;
    size_t need = align256((size_t)B * H * Sq * 4);
    // bf16 with widths and key counts that are multiples of 64 runs as tensor-core GEMMs over a score workspace
    if (dtype == FDMLA_BF16 && Skv > 0 && d_qk > 0 && d_v > 0 && d_qk % 64 == 0 && d_v % 64 == 0 && Skv % 64 == 0) {
        const size_t t = bwd_cache_latent_tensor_workspace(B, (long long)H * Sq, Skv, d_qk);
        if (t > need) need = t;
    }
    return need;
}

int fdmla_bwd_cache_latent(const void *Q, const void *K_lat, const void *O, const float *m,
                           const float *l, const void *dO, void *dQ, void *dK_lat,
                           void *workspace, size_t workspace_bytes, int B, int H, int Sq, int Skv,
                           int d_qk, int d_v, float scale, int causal, int dtype, void *stream) {
    if (!dtype_ok(dtype)) return FDMLA_ERR_INVALID;
    if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || d_qk <= 0 || d_v <= 0 || d_v > d_qk) return FDMLA_ERR_INVALID;
    if (!Q || !K_lat || !O || !m || !l || !dO || !dQ || !dK_lat) return FDMLA_ERR_INVALID;
    const size_t need = fdmla_bwd_cache_latent_workspace_bytes(B, H, Sq, Skv, d_qk, d_v, dtype);
    if (!workspace || workspace_bytes < need) return FDMLA_ERR_WORKSPACE;
    BwdProblem p{};
    p.Q = Q; p.K = K_lat; p.V = nullptr; p.O = O; p.dO = dO; p.m = m; p.l = l;
    p.D = static_cast<float *>(workspace);
    p.dQ = dQ; p.dK = dK_lat; p.dV = nullptr;
    p.G = B; p.R = H * Sq; p.Sq = Sq; p.Skv = Skv; p.d_qk = d_qk; p.d_v = d_v;
    p.causal = causal ? 1 : 0; p.scale = scale;
    if (bwd_cache_latent_tensor_supported(p, dtype)) {
        t_last_kernel = "tcgen05";
        return launch_bwd_cache_latent_tensor(p, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    }
    t_last_kernel = "portable";
    return launch_bwd_portable(p, dtype, /*grads_f32=*/0, static_cast<cudaStream_t>(stream));
}

int fdmla_cache_append(const void *new_rows, void *kv_pool, const int32_t *page_table,
                       const int32_t *start_pos, int B, int n_tokens, int d_qk, int page_size,
                       int max_pages, int num_pages, int dtype, void *stream) {
    if (!dtype_ok(dtype) || B < 0 || n_tokens < 0 || d_qk <= 0 || page_size <= 0 || max_pages < 0 || num_pages < 0)
        return FDMLA_ERR_INVALID;
    if (B == 0 || n_tokens == 0) return FDMLA_OK;
    if (!new_rows || !kv_pool || !page_table || !start_pos) return FDMLA_ERR_INVALID;
    if (B > 65535) return FDMLA_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(n_tokens, B);
    if (dtype == FDMLA_F32)
        cache_append_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float *>(new_rows),
            static_cast<float *>(kv_pool), page_table, start_pos, n_tokens, d_qk, page_size, max_pages, num_pages);
    else
        cache_append_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16 *>(new_rows),
            static_cast<__nv_bfloat16 *>(kv_pool), page_table, start_pos, n_tokens, d_qk, page_size, max_pages, num_pages);
    return check_launch();
}

int fdmla_cache_gather(const void *kv_pool, const int32_t *page_table, const int32_t *seqlens,
                       void *out, int B, int n_tokens, int d_qk, int page_size, int max_pages,
                       int num_pages, int dtype, void *stream) {
    if (!dtype_ok(dtype) || B < 0 || n_tokens < 0 || d_qk <= 0 || page_size <= 0 || max_pages < 0 || num_pages < 0)
        return FDMLA_ERR_INVALID;
    if (B == 0 || n_tokens == 0) return FDMLA_OK;
    if (!kv_pool || !page_table || !seqlens || !out) return FDMLA_ERR_INVALID;
    if (B > 65535) return FDMLA_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(n_tokens, B);
    if (dtype == FDMLA_F32)
        cache_gather_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float *>(kv_pool), page_table, seqlens,
            static_cast<float *>(out), n_tokens, d_qk, page_size, max_pages, num_pages);
    else
        cache_gather_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16 *>(kv_pool),
            page_table, seqlens, static_cast<__nv_bfloat16 *>(out), n_tokens, d_qk, page_size, max_pages, num_pages);
    return check_launch();
}

}  // extern "C"
