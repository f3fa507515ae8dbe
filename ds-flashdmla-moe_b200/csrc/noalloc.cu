// Paged decode for callers that cannot allocate device memory.
//
// Some callers of a decode step have no way to get scratch memory at call time: code that
// runs after the process has handed all device memory to a pool it does not own, plugin
// hosts that forbid allocation calls inside an operator, and callers on a path where an
// allocation would synchronise the device.  For them the split-KV partial results live in
// a fixed array that is part of the library image instead of in a caller buffer.
#include <atomic>

#include "common.cuh"

namespace fdmla {

// 32 MiB per GPU that loads the library, held until the process exits.
constexpr size_t kBuiltinScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

// The array's name is only a host-side stand-in for the symbol; the device address has to
// be asked for, once per device, with that device current.
constexpr int kMaxDevices = 64;
static std::atomic<void *> g_scratch_ptr[kMaxDevices];

static int builtin_scratch(void **ptr) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FDMLA_ERR_CUDA;
    void *p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        // two host threads may both get here; both obtain the same address
        if (cudaGetSymbolAddress(&p, g_builtin_scratch) != cudaSuccess || p == nullptr) return FDMLA_ERR_CUDA;
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *ptr = p;
    return FDMLA_OK;
}

}  // namespace fdmla

using namespace fdmla;

extern "C" {

size_t fdmla_decode_paged_noalloc_max_rows(int d_v) {
    if (d_v <= 0) return 0;
    // per partial row: d_v floats of O plus m and l, each of the three arrays 256-byte aligned
    return (kBuiltinScratchBytes - 3 * 256) / ((size_t)(d_v + 2) * sizeof(float));
}

int fdmla_decode_paged_noalloc(const void *Q, const void *kv_pool, const int32_t *page_table,
                               const int32_t *seqlens, void *O, float *m, float *l, int B, int H,
                               int d_qk, int d_v, int page_size, int max_pages, int num_pages,
                               int num_splits, float scale, int dtype, void *stream) {
    if (B < 0 || H < 0 || d_v <= 0 || num_splits < 1) return FDMLA_ERR_INVALID;
    if (!O || !m || !l) return FDMLA_ERR_INVALID;           // this variant always produces the final result
    const size_t rows = (size_t)num_splits * (size_t)B * (size_t)H;
    float *O_part = nullptr, *m_part = nullptr, *l_part = nullptr;
    if (num_splits > 1) {
        if (rows > fdmla_decode_paged_noalloc_max_rows(d_v)) return FDMLA_ERR_SCRATCH_LIMIT;
        void *base = nullptr;
        const int rc = builtin_scratch(&base);
        if (rc) return rc;
        auto align256 = [](size_t x) { return (x + 255) & ~size_t(255); };
        char *p = static_cast<char *>(base);
        O_part = reinterpret_cast<float *>(p);
        p += align256(rows * (size_t)d_v * sizeof(float));
        m_part = reinterpret_cast<float *>(p);
        p += align256(rows * sizeof(float));
        l_part = reinterpret_cast<float *>(p);
    }
    // The caller clears nothing: every partial slot a merge reads is written by the attention
    // kernel of the same call first (empty splits write l = 0), and the arrival counters of the
    // balanced schedule, which do have to start at zero, are cleared by fdmla_decode_paged with a
    // memset on the stream before its launch.
    return fdmla_decode_paged(Q, kv_pool, page_table, seqlens, O, m, l, O_part, m_part, l_part, B, H, d_qk,
                              d_v, page_size, max_pages, num_pages, num_splits, 0, -1, scale, dtype, stream);
}

}  // extern "C"
