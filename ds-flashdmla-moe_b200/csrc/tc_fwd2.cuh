// Two-CTA tensor-core Flash-DMLA forward for the MLA head dimensions
// (d_qk = 576, d_v = 512, bf16) on sm_100a.
//
// A 128-row tile (the 128 heads of a decode step, or 128 consecutive queries of
// a prefill) is owned by a CLUSTER of two CTAs running tcgen05.mma with
// cta_group::2, M = 128: each CTA holds 64 of the rows.  That is what makes the
// 512-wide output fit: 64 rows x 512 fp32 columns occupy 128 TMEM lanes x 256
// columns per CTA, next to a double-buffered S of 2 x 128 columns, and each CTA
// keeps only its 64 rows of Q (72 KB) in shared memory.
//
// Keys are processed in tiles of 256.  A tcgen05.mma costs at least ~55 cycles
// to issue whatever its shape, so every MMA here is N = 256 wide (64 cycles of
// work per SM):
//   S = Q K^T   36 MMAs per tile: for each of the 9 64-column chunks of d_qk,
//               4 K=16 steps.  A: own 64 rows of Q.  B: own 128 keys of the tile
//               x that chunk (K-major, 16 KB per CTA and chunk).
//               D: 64 rows x 256 keys -> TMEM lanes 0-63 hold keys 0-127,
//                  lanes 64-127 hold keys 128-255
//   O += P V    32 MMAs per tile: for each 64-key quarter and each half j of this
//               CTA's d_v columns, 4 K=16 steps.  A: own 64 rows of P (quarter).
//               B: the quarter's 64 keys x 128 own columns of d_v (MN-major,
//               16 KB per CTA).  D: lanes 0-63 hold d_v [0,256), lanes 64-127
//               hold d_v [256,512)
// All operand traffic goes through ONE ring of seven 16 KB slots per CTA, filled
// by TMA (no multicast anywhere) in exactly the order the MMAs consume it: Q*K^T
// of tile t+1 is issued interleaved with P*V of tile t, so the tensor pipe works on
// the next tile's scores while the softmax warps turn the current ones into P.
// Only the leader CTA (rank 0) issues MMAs; completion is
// broadcast to both CTAs' mbarriers with tcgen05.commit.  The copies of both CTAs
// credit their bytes to the leader's "slot full" barriers (cta_group::2 copies may
// name a barrier of the pair's other CTA), and both CTAs tell the leader "my P
// quarter is written" with remote mbarrier arrivals.
//
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (leader only) and TMEM
// owner, warps 2-5 softmax (thread L owns TMEM lane L: row
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

constexpr int T = 256;                // keys per tile (pair-wide)
constexpr int SUB = 64;               // keys per sub-block (one TMA box, one P quarter)
constexpr int NQC = 9;                // 64-column chunks of d_qk
constexpr int Q_CHUNK = 64 * 128;     // 64 rows x 128 B
constexpr int Q_BYTES = NQC * Q_CHUNK;            // 73 728
constexpr int SLOT = 16384;           // ring slot: 2 boxes of [64 keys x 128 B]
constexpr int BOX = 8192;
constexpr int NSLOT = 7;              // ring slots (with Q and P resident this fills the 227 KB)
constexpr int PF_DIST = 1;            // decode: how many tiles ahead the softmax threads prefetch cache rows into L2
constexpr int P_Q = 64 * SUB * 2;     // one P quarter: 64 rows x 64 keys bf16 = 8 192
constexpr int P_BYTES = 4 * P_Q;
constexpr int P_SBO = (SUB / 8) * 128;            // 1 024
constexpr int RED_BYTES = 2 * 128 * 4;
constexpr int ROWS_CACHE = 1920;      // sub-block rows resolved through the page table up front
constexpr int O_COLS = 256, S_COL0 = 256, S_COLS = 128, TMEM_COLS = 512;
// barriers (same offsets in both CTAs)
constexpr int B_QFULL = 0, B_FIXLOAD = 1, B_QEMPTY = 2, B_OFREE = 3, B_FULL = 4, B_EMPTY = B_FULL + NSLOT,
              B_FIX = B_EMPTY + NSLOT, B_SFULL = B_FIX + 1, B_SEMPTY = B_SFULL + 2, B_PFULL = B_SEMPTY + 2,
              B_OREADY = B_PFULL + 4, B_PEMPTY = B_OREADY + 2, NBARS = B_PEMPTY + 4;
constexpr int SMEM_BYTES = 1024 + Q_BYTES + NSLOT * SLOT + P_BYTES + RED_BYTES + ROWS_CACHE * 4 + NBARS * 8 + 16;
static_assert(SMEM_BYTES <= kMaxSmemPerBlock, "shared memory overflow");
constexpr int THREADS = 192;
enum { ERR_PRODUCER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_PAGE = 4, ERR_RELAY = 14,
       ERR_SOFTMAX_P = 15, ERR_SOFTMAX_RESCALE = 16, ERR_SOFTMAX_END = 17 };   // 13: scores never arrived; 15-17: P*V never completed

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Development builds only (-DFDMLA_TIMELINE): wall-clock stamps (globaltimer, ns) of what every CTA pair
// does, written by the leader CTA and dumped by the launcher to the file named by the environment variable
// FDMLA_TIMELINE_FILE after each launch.  Slot 0 kernel entry, 1 set-up done, 2 + 3 i scores of item i's first tile
// ready, 3 + 3 i item i's last P V accumulated, 4 + 3 i item i's result written, 30 roles finished, 31 exit.
// Nothing of this is compiled into the library otherwise.
#ifdef FDMLA_TIMELINE
// -DFDMLA_ABLATE=bits (with -DFDMLA_TIMELINE): time the pipeline with one stage taken out (the results are garbage).
// 1: K/V copies skipped, 2: softmax arithmetic skipped, 4: MMAs skipped.
#ifndef FDMLA_ABLATE
#define FDMLA_ABLATE 0
#endif
constexpr int ABL = FDMLA_ABLATE;
constexpr int TL_CLUSTERS = 128, TL_SLOTS = 32, TL_ITEMS = 9;
__device__ unsigned long long g_timeline[TL_CLUSTERS][TL_SLOTS];
__device__ int g_timeline_tiles[TL_CLUSTERS][TL_ITEMS];
__device__ __forceinline__ unsigned long long gtimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TL(slot) do { if (leader && cid < TL_CLUSTERS && (slot) < TL_SLOTS) g_timeline[cid][slot] = gtimer(); } while (0)
#define TL_ITEM(i, nt) do { if (leader && cid < TL_CLUSTERS && (i) < TL_ITEMS) g_timeline_tiles[cid][i] = (nt); } while (0)
// Cycles each role spends inside its waits, by kind of wait: [pair][CTA rank][role 0 producer, 1 MMA issuer / relay,
// 2 softmax thread 0][kind]; kind 7 is the role's whole loop.
constexpr int TW_KINDS = 8;
__device__ long long g_waits[TL_CLUSTERS][2][3][TW_KINDS];
constexpr int TL_TILES = 40;                                  // global-timer stamp of "scores of the pair's n-th tile are ready"
__device__ unsigned long long g_tile_ts[TL_CLUSTERS][TL_TILES];
__device__ long long g_tile_clk[TL_CLUSTERS][TL_TILES];      // SM clock at the same moments
#define TL_TILE(n) do { if (leader && cid < TL_CLUSTERS && (n) < TL_TILES) { g_tile_ts[cid][n] = gtimer(); g_tile_clk[cid][n] = clock64(); } } while (0)
#define TW_DECL long long tw[TW_KINDS] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long tw_start = clock64()
#define TW(kind, expr) ([&]() -> bool { const long long t0_ = clock64(); const bool r_ = (expr); tw[kind] += clock64() - t0_; return r_; }())
#define TW_SYNC() __syncwarp()
#define TW_BEGIN(var) const long long var = clock64()
#define TW_END(kind, var) tw[kind] += clock64() - (var)
#define TW_FLUSH(role) do { tw[7] = clock64() - tw_start; if (cid < TL_CLUSTERS) for (int k_ = 0; k_ < TW_KINDS; ++k_) g_waits[cid][rank][role][k_] = tw[k_]; } while (0)
#else
constexpr int ABL = 0;
#define TL(slot) do { } while (0)
#define TL_ITEM(i, nt) do { } while (0)
#define TL_TILE(n) do { } while (0)
#define TW_DECL do { } while (0)
#define TW(kind, expr) (expr)
#define TW_SYNC() do { } while (0)
#define TW_BEGIN(var) do { } while (0)
#define TW_END(kind, var) do { } while (0)
#define TW_FLUSH(role) do { } while (0)
#endif

// Four consecutive K=16 steps of one 2-CTA MMA: descriptors advance by a_step / b_step (in
// 16-byte units of the start-address field) per step.  acc0 == 0 makes the first step overwrite D.
__device__ __forceinline__ void mma4_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t a_step,
                                          uint32_t b_step, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 sa, sb, a1, a2, a3, b1, b2, b3;\n"
        "setp.ne.b32 p, %6, 0;\n"
        "cvt.u64.u32 sa, %3;\n"
        "cvt.u64.u32 sb, %4;\n"
        "add.s64 a1, %1, sa;\n add.s64 a2, a1, sa;\n add.s64 a3, a2, sa;\n"
        "add.s64 b1, %2, sb;\n add.s64 b2, b1, sb;\n add.s64 b3, b2, sb;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %5, p;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a1, b1, %5, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a2, b2, %5, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a3, b3, %5, 1;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(a_step), "r"(b_step), "r"(idesc), "r"(acc0)
        : "memory");
}

// P quarters are produced in the order (0, 2), (1, 3) - the two key halves of a tile work side by
// side - and P*V consumes them in that order, so that half of a tile's P*V is out of the way
// before the second pair of quarters is even written.
__device__ __forceinline__ int quarter_at(int i) { return ((i & 1) << 1) | (i >> 1); }      // 0, 2, 1, 3

// Ring slots are filled and consumed in one order: the nine K slots of tile 0, then for every tile t the three K
// slot groups of tile t + 1 (its Q K^T runs while the softmax of tile t works) interleaved with the V slot pairs of
// tile t's quarters in the order of quarter_at: K group 0, V pair, K group 1, V pair, K group 2, V pair, V pair.
// Slots then come free at a steady rate (3, 2, 3, 2, 3, 2, 2 instead of nine and then eight), which measured 3 %
// faster in decode and 8 % faster in prefill than the whole K tile followed by the whole V tile.

// Keys of KV group g.  A length outside [0, Skv] (Skv = max_pages * page_size for a paged cache) is clamped:
// the page table has no entries for more, and an unclamped length would cut a sequence into more pieces
// than the caller's scratch has slabs for.  The producer reports the clamp through the error flag.
__device__ __forceinline__ int group_seq(const FwdProblem &p, int g) {
    if (!p.seqlens) return p.Skv;
    const int s = p.seqlens[g];
    return s < 0 ? 0 : (s > p.Skv ? p.Skv : s);
}

// One unit of work of the persistent kernel: a 128-row tile of one KV group and one KV split.
struct Item {
    int row0, g, split;       // first row of the tile, KV group, split index
    int seq;                  // keys of the group
    int lo, hi;               // this split's key window
    int blk_hi;               // end of the keys any row of the tile may see
    int t_begin;              // first key of the first tile (lo rounded down to a tile)
    int n_sub, n_tiles;       // 64-key sub-blocks / 256-key tiles to attend
    int rows_here;
    bool fix;                 // the last sub-block reaches past the end of the sequence (its V rows get zeroed)
    bool final_out;           // the item covers every key of its rows: write O, m, l instead of a partial
    int n_parts;              // balanced schedule: pieces the sequence is cut into (0 otherwise)
};

__device__ __forceinline__ Item make_item(const FwdProblem &p, int idx, int n_row_tiles, bool poisoned) {
    Item it;
    const int per_rt = p.G * p.num_splits;
    const int rt = idx / per_rt, rem = idx - rt * per_rt;
    it.g = rem / p.num_splits;
    it.split = rem - it.g * p.num_splits;
    const int tile_idx = p.causal ? n_row_tiles - 1 - rt : rt;     // causal: the longest rows first
    it.row0 = tile_idx * 128;
    it.seq = group_seq(p, it.g);
    const int w_lo = p.kv_begin > 0 ? p.kv_begin : 0;
    const int w_hi = (p.kv_end >= 0 && p.kv_end < it.seq) ? p.kv_end : it.seq;
    // splits are cut on tile boundaries where the page size allows it
    const int gran = (p.page_table && (T % p.page_size) != 0) ? p.page_size : T;
    split_window(w_lo, w_hi, gran, it.split, p.num_splits, &it.lo, &it.hi);
    it.rows_here = (p.R - it.row0) < 128 ? (p.R - it.row0) : 128;
    int blk_vis = it.seq;
    if (p.causal) {
        const int r_last = it.row0 + it.rows_here - 1;
        const int i_max = (it.row0 / p.Sq == r_last / p.Sq) ? (r_last % p.Sq) : (p.Sq - 1);
        long long v = (long long)i_max + it.seq - p.Sq + 1;
        blk_vis = v < 0 ? 0 : (v > it.seq ? it.seq : (int)v);
    }
    it.blk_hi = it.hi < blk_vis ? it.hi : blk_vis;
    it.t_begin = (it.lo / T) * T;
    it.n_sub = (it.blk_hi > it.lo && !poisoned) ? (it.blk_hi - it.t_begin + SUB - 1) / SUB : 0;
    it.n_tiles = (it.n_sub + 3) / 4;
    it.fix = it.n_sub > 0 && it.t_begin + it.n_sub * SUB > it.seq;
    it.final_out = p.num_splits == 1 && p.O != nullptr;
    it.n_parts = 0;
    return it;
}

// The persistent grid walks one of two schedules.
//  * Items: cluster c takes items c, 2n-1-c, 2n+c, ... (a snake over rounds of n clusters, so that an
//    order sorted by work does not always hand the same cluster the largest item of a round).
//  * Balanced (decode with a final output and spare partial slabs): the 256-key tiles of all sequences
//    are laid end to end (an empty sequence counts as one) and cluster c takes tiles [c q, (c+1) q) of that
//    line, q = max(ceil(total / n), quota_min).  A sequence that lies inside one cluster's run is
//    written as the final result; one that is cut is written as partials (piece k into slab k) and merged
//    either by the pair that finishes the sequence's last piece (p.tickets != nullptr) or by a second
//    kernel.  quota_min bounds the pieces per sequence by the number of slabs.
//    A run is walked last sequence first, then the others in order: the sequences a run shares with its
//    neighbours come first, so that both halves of a cut sequence are finished early in their runs and
//    the merge of the pair that arrives second is not what the kernel ends with.
struct Cursor {
    bool balanced;
    // items
    int round, n_rounds, cid, n_clusters, n_items, n_row_tiles;
    // balanced
    int quota, run_lo, run_hi;                 // this cluster's tiles [run_lo, run_hi) on the line
    int g_last, first_of_last;                 // sequence holding tile run_hi - 1 and the position of its first tile
    int g, first_of_g;                         // walking state: next sequence in order and its first tile
    int g_end;                                 // the in-order walk stops before this sequence
    int phase;                                 // 0: the last sequence is due, 1: the others in order, 2: done
};

__device__ __forceinline__ int sched_tiles(const FwdProblem &p, int g) {
    const int nt = (group_seq(p, g) + T - 1) / T;
    return nt > 0 ? nt : 1;
}

// Sequence holding tile `pos` of the line and the position of that sequence's first tile.  Called by all 32
// lanes of a warp together; pos must be below the line's length.
__device__ __forceinline__ void line_locate(const FwdProblem &p, int pos, int lane, int &g, int &first) {
    int base = 0;
    g = p.G - 1; first = 0;
    for (int g0 = 0; g0 < p.G; g0 += 32) {
        const int v = (g0 + lane < p.G) ? sched_tiles(p, g0 + lane) : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, (g0 + lane < p.G) && base + incl > pos);
        if (hit) {
            const int src = __ffs(hit) - 1;
            first = __shfl_sync(0xffffffffu, base + incl - v, src);
            g = g0 + src;
            return;
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
}

// Called by all 32 lanes of a warp together.
template <bool DECODE>
__device__ __forceinline__ void cursor_init(Cursor &c, const FwdProblem &p, int cid, int n_clusters, int lane) {
    c.balanced = DECODE && p.balanced != 0;
    c.cid = cid;
    c.n_clusters = n_clusters;
    c.round = 0;
    c.n_row_tiles = (p.R + 127) / 128;
    c.n_items = c.n_row_tiles * p.G * p.num_splits;
    c.n_rounds = (c.n_items + n_clusters - 1) / n_clusters;
    c.quota = 1; c.run_lo = c.run_hi = 0; c.g_last = c.first_of_last = c.g = c.first_of_g = c.g_end = 0; c.phase = 2;
    if (!c.balanced) return;
    int total = 0;
    for (int g0 = 0; g0 < p.G; g0 += 32) total += (g0 + lane < p.G) ? sched_tiles(p, g0 + lane) : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    int q = (total + n_clusters - 1) / n_clusters;
    if (q < p.quota_min) q = p.quota_min;
    if (q < 1) q = 1;
    c.quota = q;
    const long long start_ll = (long long)cid * q;
    if (start_ll >= total) return;                    // nothing left for this cluster
    c.run_lo = (int)start_ll;
    c.run_hi = (total - c.run_lo) < q ? total : c.run_lo + q;
    line_locate(p, c.run_lo, lane, c.g, c.first_of_g);
    line_locate(p, c.run_hi - 1, lane, c.g_last, c.first_of_last);
    c.phase = (c.g_last != c.g) ? 0 : 1;
    c.g_end = (c.g_last != c.g) ? c.g_last : c.g_last + 1;
}

// Next item of this cluster (the same in every thread that asks); false when the cluster is done.
__device__ __forceinline__ bool cursor_next(Cursor &c, const FwdProblem &p, bool poisoned, Item &it) {
    if (!c.balanced) {
        while (c.round < c.n_rounds) {
            const int idx = c.round * c.n_clusters + ((c.round & 1) ? c.n_clusters - 1 - c.cid : c.cid);
            ++c.round;
            if (idx < c.n_items) { it = make_item(p, idx, c.n_row_tiles, poisoned); return true; }
        }
        return false;
    }
    if (c.phase >= 2) return false;
    int g, first;
    if (c.phase == 0) {
        g = c.g_last; first = c.first_of_last; c.phase = 1;
    } else {
        if (c.g >= c.g_end) { c.phase = 2; return false; }
        g = c.g; first = c.first_of_g;
    }
    const int seq = group_seq(p, g);
    const int nt = sched_tiles(p, g);
    if (g == c.g) { c.first_of_g += nt; ++c.g; }        // the in-order walk moves on
    // tiles of this sequence inside the run
    const int a = first > c.run_lo ? first : c.run_lo, b = (first + nt) < c.run_hi ? (first + nt) : c.run_hi;
    const int ta = a - first, tb = b - first;
    it.row0 = 0; it.g = g; it.seq = seq;
    it.lo = ta * T;
    it.hi = tb * T < seq ? tb * T : seq;
    if (it.hi < it.lo) it.hi = it.lo;
    it.blk_hi = it.hi;
    it.t_begin = it.lo;
    it.rows_here = p.R < 128 ? p.R : 128;
    it.n_sub = (it.hi > it.lo && !poisoned) ? (it.hi - it.lo + SUB - 1) / SUB : 0;
    it.n_tiles = (it.n_sub + 3) / 4;
    it.fix = it.n_sub > 0 && it.t_begin + it.n_sub * SUB > seq;
    it.final_out = ta == 0 && tb == nt && p.balanced != 2;      // balanced == 2: partials only, nothing is final
    it.split = c.cid - first / c.quota;                         // piece index within the sequence
    it.n_parts = (first + nt - 1) / c.quota - first / c.quota + 1;
    return true;
}

// DECODE (one query token per KV group row set): L2 prefetch, TMA-store epilogue and the balanced schedule
// are compiled in; the prefill instantiation carries none of them.
template <bool DECODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
fwd_tc2_kernel(const FwdProblem p, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO) {
    // tmQ: chunked view, box {64, 64 rows, 9 chunks}; tmK: plain 2-D, box {64, 64 rows};
    // tmV: chunked view of the same cache, box {64, 64 rows, 2 chunks};
    // tmO: the bf16 output [G R, 512], box {64, 64 rows} (a copy of tmK when there is no final output)
    using namespace ptx;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sQ = smem;
    uint8_t *sRing = sQ + Q_BYTES;                     // [NSLOT][2 boxes][64 keys][128 B]
    uint8_t *sP = sRing + NSLOT * SLOT;                // [4 quarters][64 rows x 64 keys bf16]
    float *red = reinterpret_cast<float *>(sP + P_BYTES);       // [2][128]
    int *s_rows = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(red) + RED_BYTES);   // [ROWS_CACHE]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_rows + ROWS_CACHE);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    int *err_slot = reinterpret_cast<int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;

    // ---- the work list (identical in both CTAs of the pair and in every role) -----------
    const int cid = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    if (threadIdx.x == 0) TL(0);

    // ---- set-up ------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        *err_slot = *reinterpret_cast<volatile int *>(&g_tc_error);
        mbar_init(BAR(B_QFULL), 1);          // leader: its producer's arrival, the bytes of both CTAs' copies
        mbar_init(BAR(B_FIXLOAD), 1);        // own copies of a V slot pair whose tail has to be zeroed
        mbar_init(BAR(B_QEMPTY), 1);
        mbar_init(BAR(B_OFREE), 2);                      // one arrival per CTA of the pair
        for (int s = 0; s < NSLOT; ++s) {
            mbar_init(BAR(B_FULL + s), 1);    // used in the leader only: both CTAs' copies credit their bytes to it
            mbar_init(BAR(B_EMPTY + s), 1);
        }
        mbar_init(BAR(B_FIX), 2);          // leader: both CTAs have zero-filled the tail of a V slot pair (once per item at most)
        for (int b = 0; b < 2; ++b) {
            mbar_init(BAR(B_SFULL + b), 1);
            mbar_init(BAR(B_SEMPTY + b), 4);     // two key halves in each CTA of the pair
            mbar_init(BAR(B_OREADY + b), 1);
        }
        for (int q = 0; q < 4; ++q) {
            mbar_init(BAR(B_PFULL + q), 2);    // one arrival per CTA
            mbar_init(BAR(B_PEMPTY + q), 1);   // P*V of that quarter has read it
        }
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
    // Once any CTA has reported a failed wait the rest of the grid does no work.  The leader's thread 0 has read the
    // flag once (before the barriers above); every thread of the pair takes that one value from the leader's shared
    // memory, so that all roles of both CTAs walk the same item list even if the flag changes meanwhile.
    const int err_now = (int)ld_shared_cluster_u32(map_to_cta(smem_u32(err_slot), 0));
    const bool poisoned = err_now != 0 && err_now != ERR_PAGE;
    if (threadIdx.x == 0) TL(1);

    // global row of the first key of sub-block s of an item (pool row for paged caches)
    auto sub_row = [&](const Item &it, int s, bool *bad_page) -> int {
        const int t0 = it.t_begin + s * SUB;
        if (p.page_table) {
            const int lp = t0 / p.page_size;
            int pg = lp < p.max_pages ? p.page_table[(size_t)it.g * p.max_pages + lp] : -1;
            if (pg < 0 || pg >= p.num_pages) { *bad_page = true; pg = 0; }
            return pg * p.page_size + (t0 - lp * p.page_size);
        }
        return it.g * p.Skv + t0;
    };

    // Every role walks the same items in the same order and keeps its own running counts of the
    // things whose barrier phases span items: ring position, tiles (S/P/O barriers), items that
    // loaded a Q (Q barriers), items (O-free barrier) and uses of the tail-fix barriers.
    if (warp == 0) {
        // =========================== TMA producer (both CTAs) ============================
        bool bad = false, ok = true;
        const bool elected = elect_one();
        int next_slot = 0, next_use = 0;      // ring position and how many times the ring has wrapped
        int q_loads = 0, fix_uses = 0;
        // Every copy of the pair credits its bytes to a barrier of the LEADER CTA (cta_group::2 copies may name a
        // barrier of the other CTA of the pair): the MMA issuer then waits on one barrier per slot for both halves,
        // and the leader's producer announces the bytes of both CTAs.
        const uint32_t lead_bars = map_to_cta(bar0, 0);
        TW_DECL;
        if (lane == 0) {
            prefetch_tmap(&tmQ);
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
        }
        Cursor cur;
        cursor_init<DECODE>(cur, p, cid, n_clusters, lane);
        Item it;
        for (int round = 0; ok && cursor_next(cur, p, poisoned, it); ++round) {
            if (p.seqlens && p.seqlens[it.g] != it.seq) bad = true;      // a length outside [0, max_pages * page_size] was clamped
            if (it.n_tiles == 0) continue;
            // Q of the previous item is free once its last Q K^T has completed
            if (q_loads > 0) ok = ok && TW(0, mbar_wait(BAR(B_QEMPTY), (q_loads - 1) & 1));
            TW_BEGIN(tw_set);
            if (elected) {
                if (leader) mbar_arrive_expect_tx(BAR(B_QFULL), 2 * Q_BYTES);       // this CTA's rows and the peer's
                const int qrow = it.g * p.R + it.row0 + 64 * (int)rank;
                tma_load_3d_pair(smem_u32(sQ), &tmQ, 0, qrow, 0, lead_bars + 8u * B_QFULL);   // all 9 chunks in one copy
            }
            ++q_loads;
            // resolve the page table for the whole key range once, with every lane of the warp
            const int n_cached = it.n_sub < ROWS_CACHE ? it.n_sub : ROWS_CACHE;
            __syncwarp();
            for (int s = lane; s < n_cached; s += 32) s_rows[s] = sub_row(it, s, &bad);
            __syncwarp();
            auto row_of = [&](int s) -> int { return s < ROWS_CACHE ? s_rows[s] : sub_row(it, s, &bad); };
            TW_END(6, tw_set);
            // The whole warp walks the ring converged and one elected lane issues the copies (the
            // uniform datapath makes the issue several times cheaper than from a lone diverged lane).
            auto take = [&](int &slot, int &use) {
                slot = next_slot; use = next_use;
                if (++next_slot == NSLOT) { next_slot = 0; ++next_use; }
            };
            // three K slots: chunks 3*g3 .. 3*g3+2 of K tile t (own 128 keys = two sub-blocks each)
            auto fill_k3 = [&](int t, int g3) {
                int sl[3], us[3];
                for (int i = 0; i < 3; ++i) take(sl[i], us[i]);
                if (us[2] >= 1) {     // slots handed out before: wait until the MMAs that read them are done
                    if (us[0] >= 1)
                        ok = ok && TW(1, mbar_wait3(BAR(B_EMPTY + sl[0]), (us[0] - 1) & 1, BAR(B_EMPTY + sl[1]), (us[1] - 1) & 1,
                                              BAR(B_EMPTY + sl[2]), (us[2] - 1) & 1));
                    else if (us[1] >= 1)
                        ok = ok && TW(1, mbar_wait2(BAR(B_EMPTY + sl[1]), (us[1] - 1) & 1, BAR(B_EMPTY + sl[2]), (us[2] - 1) & 1));
                    else
                        ok = ok && TW(1, mbar_wait(BAR(B_EMPTY + sl[2]), (us[2] - 1) & 1));
                }
                auto present_of = [&](int s_first) { return (s_first + 1 < it.n_sub) ? 2 : (s_first < it.n_sub ? 1 : 0); };
                const int s0 = 4 * t + 2 * (int)rank;
                const int present = present_of(s0);
                const int present_pair = present_of(4 * t) + present_of(4 * t + 2);
                const int r0 = present > 0 ? row_of(s0) : 0, r1 = present > 1 ? row_of(s0 + 1) : 0;
                TW_BEGIN(tw_ki);
                if (elected) {
#pragma unroll
                    for (int i = 0; i < 3; ++i) {
                        const uint32_t full = lead_bars + 8u * (B_FULL + sl[i]);
                        const uint32_t dst = smem_u32(sRing + sl[i] * SLOT);
                        if (ABL & 1) { if (leader) mbar_arrive(BAR(B_FULL + sl[i])); continue; }
                        if (leader) mbar_arrive_expect_tx(BAR(B_FULL + sl[i]), present_pair * BOX);
                        if (present > 0) tma_load_2d_pair(dst, &tmK, (3 * g3 + i) * 64, r0, full);
                        if (present > 1) tma_load_2d_pair(dst + BOX, &tmK, (3 * g3 + i) * 64, r1, full);
                    }
                }
                TW_SYNC();
                TW_END(4, tw_ki);
            };
            // two V slots: the 64 keys of quarter q of tile t, own d_v columns [256 r + 128 j, +128), j = 0, 1
            auto fill_v2 = [&](int t, int q) {
                int sl[2], us[2];
                for (int j = 0; j < 2; ++j) take(sl[j], us[j]);
                if (us[0] >= 1)
                    ok = ok && TW(2, mbar_wait2(BAR(B_EMPTY + sl[0]), (us[0] - 1) & 1, BAR(B_EMPTY + sl[1]), (us[1] - 1) & 1));
                else if (us[1] >= 1)
                    ok = ok && TW(2, mbar_wait(BAR(B_EMPTY + sl[1]), (us[1] - 1) & 1));
                const int s = 4 * t + q;
                const int row = row_of(s);
                const int t0 = it.t_begin + s * SUB;
                const bool tail = t0 + SUB > it.seq;      // keys past the end of the sequence in this sub-block
                TW_BEGIN(tw_vi);
                if (elected) {
                    if (!tail) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (ABL & 1) { if (leader) mbar_arrive(BAR(B_FULL + sl[j])); continue; }
                            if (leader) mbar_arrive_expect_tx(BAR(B_FULL + sl[j]), 2 * SLOT);
                            tma_load_3d_pair(smem_u32(sRing + sl[j] * SLOT), &tmV, 0, row, 4 * (int)rank + 2 * j,
                                             lead_bars + 8u * (B_FULL + sl[j]));   // two chunks, one copy
                        }
                    } else {
                        // the copies of this pair of slots report to a barrier of this CTA, which has to touch the data
                        // before the MMAs may; the slots' own barriers complete their phase without bytes
                        mbar_arrive_expect_tx(BAR(B_FIXLOAD), 2 * SLOT);
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (leader) mbar_arrive(BAR(B_FULL + sl[j]));
                            tma_load_3d(smem_u32(sRing + sl[j] * SLOT), &tmV, 0, row, 4 * (int)rank + 2 * j, BAR(B_FIXLOAD));
                        }
                    }
                }
                TW_SYNC();
                TW_END(5, tw_vi);
                if (tail) {
                    // zero the V rows of the keys past the end once the copies have landed (whole 128-byte rows,
                    // so the swizzle does not matter), then tell the leader's MMA issuer
                    ok = ok && TW(3, mbar_wait(BAR(B_FIXLOAD), fix_uses & 1));
                    const int first_bad = it.seq > t0 ? it.seq - t0 : 0;
                    const int bad_rows = SUB - first_bad;
                    for (int idx2 = lane; idx2 < 4 * bad_rows * 8; idx2 += 32) {
                        const int cc = idx2 / (bad_rows * 8), rem = idx2 - cc * bad_rows * 8;
                        *reinterpret_cast<uint4 *>(sRing + sl[cc >> 1] * SLOT + (cc & 1) * BOX + (first_bad + rem / 8) * 128 +
                                                   (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (elected) mbar_arrive_cluster(lead_bars + 8u * B_FIX);   // (release, cluster scope: once per item at most)
                    ++fix_uses;                                                // only the last sub-block of an item can straddle the end
                }
            };
            for (int g3 = 0; g3 < 3; ++g3) fill_k3(0, g3);
            for (int t = 0; t < it.n_tiles && ok; ++t) {
                const int nq = (it.n_sub - 4 * t) < 4 ? (it.n_sub - 4 * t) : 4;
                const bool more = t + 1 < it.n_tiles;
for (int i = 0; i < 4; ++i) {
                    if (i < 3 && more) fill_k3(t + 1, i);
                    if (quarter_at(i) < nq) fill_v2(t, quarter_at(i));
                }
            }
        }
        if (lane == 0) TW_FLUSH(0);
        if (!ok && lane == 0) atomicCAS(&g_tc_error, 0, ERR_PRODUCER);
        if (bad) atomicCAS(&g_tc_error, 0, ERR_PAGE);
        __syncwarp();
    } else if (warp == 1) {
        if (leader) {
            // =========================== MMA issuer (leader CTA) =========================
            // The whole warp runs this loop converged and one elected lane issues: that keeps the
            // descriptor arithmetic on the uniform datapath, which is what lets tcgen05.mma issue at
            // full rate (a single diverged lane issuing the same sequence is about half as fast).
            const bool elected = elect_one();
            constexpr uint32_t idesc_qk = make_idesc_bf16(128, 256, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_bf16(128, 256, 0, 1);
            const uint64_t q_desc = make_smem_desc(smem_u32(sQ), 16, 1024, kLayoutSw128);
            const uint64_t rk_desc = make_smem_desc(smem_u32(sRing), 16, 1024, kLayoutSw128);    // ring slot as K-major B
            const uint64_t rv_desc = make_smem_desc(smem_u32(sRing), BOX, 1024, kLayoutSw128);   // ring slot as MN-major B
            const uint64_t p_desc = make_smem_desc(smem_u32(sP), 128, P_SBO, kLayoutNone);
            bool ok = true;
            int slot = 0;               // ring position (the same in every lane) and its phase
            uint32_t ph = 0;
            int tg0 = 0;                // tiles of the items before the current one
            int q_loads = 0, items_done = 0, fix_uses = 0;     // items_done: items that used the accumulator
            TW_DECL;
            Cursor cur;
            cursor_init<DECODE>(cur, p, cid, n_clusters, lane);
            Item it;
            for (int round = 0; cursor_next(cur, p, poisoned, it); ++round) {
                if (!__all_sync(0xffffffffu, ok)) break;
                if (it.n_tiles == 0) continue;       // nothing to multiply; the softmax warps write the empty result
                // The accumulator is needed again only after the softmax warps of both CTAs have read the
                // previous item's O out of tensor memory.
                bool o_free_waited = items_done == 0;
                auto wait_o_free = [&]() {
                    if (!o_free_waited) {
                        ok = ok && TW(6, mbar_wait(BAR(B_OFREE), (items_done - 1) & 1));
                        tc_fence_after_sync();
                        o_free_waited = true;
                    }
                };
                ok = ok && TW(0, mbar_wait(BAR(B_QFULL), q_loads & 1));
                ++q_loads;
                auto take = [&](int &sl, uint32_t &pp) {
                    sl = slot; pp = ph;
                    if (++slot == NSLOT) { slot = 0; ph ^= 1; }
                };
                // S = Q K^T: chunks 3*g3 .. 3*g3+2 of K tile tk, three ring slots waited for together
                auto k_group = [&](int tk, int g3) {
                    const int tg = tg0 + tk, b = tg & 1;
                    int sl[3];
                    uint32_t phs[3];
                    for (int i = 0; i < 3; ++i) take(sl[i], phs[i]);
                    if (g3 == 0) {
                        // S[b] was last read by the softmax of the tile two before
                        if (tg >= 2) ok = ok && TW(1, mbar_wait(BAR(B_SEMPTY + b), ((tg / 2) - 1) & 1));
                        tc_fence_after_sync();
                    }
#pragma unroll
                    for (int i = 0; i < 3; ++i) {
                        // (waiting slot by slot measured 2 % faster than waiting for the three together)
                        ok = ok && TW(2, mbar_wait(BAR(B_FULL + sl[i]), phs[i]));
                        if (elected) {
                            const int c = 3 * g3 + i;
                            if (!(ABL & 4)) mma4_2cta(tmem + S_COL0 + b * S_COLS, q_desc + (uint32_t)c * (Q_CHUNK >> 4),
                                      rk_desc + (uint32_t)sl[i] * (SLOT >> 4), 2, 2, idesc_qk, c != 0);
                            mma_commit_2cta(BAR(B_EMPTY + sl[i]), 3);
                        }
                    }
                    if (elected) {
                        if (g3 == 2) {
                            mma_commit_2cta(BAR(B_SFULL + b), 3);
                            if (tk == it.n_tiles - 1) mma_commit_2cta(BAR(B_QEMPTY), 3);   // last use of this item's Q
                        }
                    }
                };
                // O += P V: quarter q of tile t, both halves j of this CTA's d_v columns
                auto v_pair = [&](int t, int q, bool last) {
                    const int tg = tg0 + t;
                    int sl[2];
                    uint32_t phs[2];
                    for (int j = 0; j < 2; ++j) take(sl[j], phs[j]);
                    ok = ok && TW(3, mbar_wait(BAR(B_PFULL + q), tg & 1));
                    tc_fence_after_sync();      // orders the accumulation after the softmax's rescale of O
                    ok = ok && TW(4, mbar_wait2(BAR(B_FULL + sl[0]), phs[0], BAR(B_FULL + sl[1]), phs[1]));
                    if (it.t_begin + (4 * t + q) * SUB + SUB > it.seq)
                        ok = ok && TW(5, mbar_wait_cluster(BAR(B_FIX), fix_uses & 1));
                    if (elected) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (!(ABL & 4)) mma4_2cta(tmem + j * 128, p_desc + (uint32_t)q * (P_Q >> 4), rv_desc + (uint32_t)sl[j] * (SLOT >> 4),
                                      16, 128, idesc_pv, (t | q) != 0);
                            mma_commit_2cta(BAR(B_EMPTY + sl[j]), 3);
                        }
                        mma_commit_2cta(BAR(B_PEMPTY + q), 3);    // this P quarter may be overwritten
                        if (last) mma_commit_2cta(BAR(B_OREADY + (tg & 1)), 3);   // tile t folded into O
                    }
                };
#pragma unroll
                for (int g3 = 0; g3 < 3; ++g3) k_group(0, g3);
#pragma unroll 1
                for (int t = 0; t < it.n_tiles; ++t) {
                    if (!__all_sync(0xffffffffu, ok)) break;
                    const int nq = (it.n_sub - 4 * t) < 4 ? (it.n_sub - 4 * t) : 4;
                    const int q_last = nq == 3 ? 1 : nq - 1;       // last quarter in the order 0, 2, 1, 3
                    const bool more = t + 1 < it.n_tiles;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (i < 3 && more) k_group(t + 1, i);
                        if (t == 0 && i == 0) wait_o_free();     // the first P V of the item overwrites O
                        const int q = quarter_at(i);
                        if (q < nq) v_pair(t, q, q == q_last);
                    }
                }
                tg0 += it.n_tiles;
                fix_uses += it.fix ? 1 : 0;
                ++items_done;
            }
            if (lane == 0) TW_FLUSH(1);
            if (!ok && lane == 0) atomicCAS(&g_tc_error, 0, ERR_MMA);
        }
        // (warp 1 of the peer CTA only owns the tensor-memory allocation: every copy of the pair reports to the
        // leader's barriers by itself)
        __syncwarp();
    } else {
        // =========================== softmax + epilogue (both CTAs) ========================
        const int L = (warp & 3) * 32 + lane;          // TMEM lane owned by this thread
        const int row = L & 63, half = L >> 6;         // key half: keys [128 half, +128) of every tile
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;
        const uint32_t pfull_leader = map_to_cta(BAR(B_PFULL), 0);
        const uint32_t sempty_leader = map_to_cta(BAR(B_SEMPTY), 0);
        const uint32_t ofree_leader = map_to_cta(BAR(B_OFREE), 0);
        constexpr bool do_prefetch = DECODE;    // decode streams the cache from HBM; prefill finds it in L2 anyway
        bool ok = true;
        int fail = 0;                           // which wait gave up first
        // P*V passes that have read this thread's two P quarters so far (a quarter past the end of the
        // keys is written - as zeros - but never read): the phase to wait for before overwriting one
        int p_reads[2] = {0, 0};
        int tg0 = 0;                            // tiles of the items before the current one
        uint32_t r[32];
        TW_DECL;
        Cursor cur;
        cursor_init<DECODE>(cur, p, cid, n_clusters, lane);
        Item it;
        for (int round = 0; cursor_next(cur, p, poisoned, it); ++round) {
            const int rr = it.row0 + 64 * (int)rank + row;
            const bool row_ok = rr < p.R;
            const int lo = it.lo, hi = it.hi, seq = it.seq, n_tiles = it.n_tiles;
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
            float m_true = -CUDART_INF_F, m_ref = -CUDART_INF_F, l_run = 0.f;   // l_run: this thread's key half only
            // decode: the cache row this thread pulls into L2 for the first tile of the pair's NEXT item while it works
            // on the last tile of this one (an item's first tile has no tile before it to do that)
            const char *next_first_row = nullptr;
            if (do_prefetch && PF_DIST > 0 && n_tiles > 0) {
                Cursor peek = cur;
                Item nxt;
                while (cursor_next(peek, p, poisoned, nxt))
                    if (nxt.n_tiles > 0) {
                        const int s = 2 * (int)rank + half;
                        bool bad_page = false;
                        if (s < nxt.n_sub && nxt.t_begin + s * SUB + row < nxt.blk_hi) {
                            const size_t r0 = (size_t)sub_row(nxt, s, &bad_page) + row;
                            if (!bad_page) next_first_row = static_cast<const char *>(p.K) + r0 * (NQC * 128);
                        }
                        break;
                    }
            }
            for (int t = 0; t < n_tiles; ++t) {
                const int tg = tg0 + t, b = tg & 1, tok0 = it.t_begin + t * T + 128 * half;
                const uint32_t s_addr = tmem + lane_base + S_COL0 + b * S_COLS;
                // after a failed wait the loop keeps running without further waits so that the
                // named barriers below stay matched across the softmax threads
                if (PF_DIST > 0 && do_prefetch) {
                    // While this thread would only wait for S: pull one cache row of a later tile into L2.
                    // The 128 softmax threads of the CTA cover the CTA's own 128 keys of that tile (the
                    // pair covers the tile), so the TMA copies issued PF_DIST tiles from now hit L2 and
                    // the ring only has to hide the L2 latency, not the HBM latency.
                    if (t == n_tiles - 1 && next_first_row != nullptr) {
#pragma unroll
                        for (int c = 0; c < NQC; ++c) prefetch_l2(next_first_row + c * 128);
                    }
                    for (int tp = (t == 0 ? 1 : t + PF_DIST); tp <= t + PF_DIST; ++tp) {
                        const int s = 4 * tp + 2 * (int)rank + half;
                        if (s < it.n_sub && it.t_begin + s * SUB + row < it.blk_hi) {
                            bool bad_page = false;
                            const char *src = static_cast<const char *>(p.K) + ((size_t)sub_row(it, s, &bad_page) + row) * (NQC * 128);
                            if (!bad_page) {
#pragma unroll
                                for (int c = 0; c < NQC; ++c) prefetch_l2(src + c * 128);
                            }
                        }
                    }
                }
                if (ok && !(ok = TW(0, mbar_wait(BAR(B_SFULL + b), (tg / 2) & 1)))) fail = ERR_SOFTMAX;
                if (L == 0 && t == 0) TL(2 + 3 * round);
                if (L == 0) TL_TILE(tg);
                tc_fence_after_sync();
                // pass 1: maximum of this thread's 128 keys (no per-key masking when all are visible)
                const bool all_visible = tok0 >= lo && tok0 + 128 <= upper && sl2 > 0.f;
                float tmax = -CUDART_INF_F;
#pragma unroll 1
                for (int cp = (ABL & 2) ? 4 : 0; cp < 4; cp += 2) {
                    // two 32-column loads in flight per wait
                    uint32_t r2[32];
                    tmem_ld32(s_addr + cp * 32, r);
                    tmem_ld32(s_addr + (cp + 1) * 32, r2);
                    tmem_wait_ld();
                    if (all_visible) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) tmax = fmaxf(tmax, fmaxf(__uint_as_float(r[j]), __uint_as_float(r2[j])));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int tok = tok0 + cp * 32 + j;
                            if (tok >= lo && tok < upper) tmax = fmaxf(tmax, __uint_as_float(r[j]) * sl2);
                            if (tok + 32 >= lo && tok + 32 < upper) tmax = fmaxf(tmax, __uint_as_float(r2[j]) * sl2);
                        }
                    }
                }
                if (all_visible) tmax *= sl2;     // fast path took the maximum of the raw scores (sl2 > 0)
                // the row's other key half lives in the thread 64 lanes away
                red[(tg & 1) * 128 + L] = tmax;
                named_bar_sync(1, 128);
                tmax = fmaxf(tmax, red[(tg & 1) * 128 + (L ^ 64)]);
                const float m_new = fmaxf(m_true, tmax);
                const bool need = m_new > m_ref + 8.f;
                if (__any_sync(0xffffffffu, need)) {
                    // O is rescaled: every P*V of tile t-1 must have been accumulated
                    if (t > 0) {
                        if (ok && !(ok = TW(1, mbar_wait(BAR(B_OREADY + ((tg - 1) & 1)), ((tg - 1) / 2) & 1)))) fail = ERR_SOFTMAX_RESCALE;
                        tc_fence_after_sync();
                    }
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
                // pass 2: P = 2^(s - m_ref), quarter by quarter (this half owns quarters 2*half, 2*half+1)
                float lsum = 0.f;
#pragma unroll 1
                for (int cc = 0; cc < 4; ++cc) {
                    if (!(ABL & 2)) {
                        tmem_ld32(s_addr + cc * 32, r);
                        tmem_wait_ld();
                    }
                    uint32_t packed[16];
                    if (ABL & 2) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) packed[j] = 0;
                    } else if (all_visible) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float p0 = fast_exp2(fmaf(__uint_as_float(r[j]), sl2, -m_ref));
                            const float p1 = fast_exp2(fmaf(__uint_as_float(r[j + 1]), sl2, -m_ref));
                            lsum += p0 + p1;
                            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                            packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const int tok = tok0 + cc * 32 + j;
                            const float p0 = (tok >= lo && tok < upper) ? fast_exp2(fmaf(__uint_as_float(r[j]), sl2, -m_ref)) : 0.f;
                            const float p1 = (tok + 1 >= lo && tok + 1 < upper) ? fast_exp2(fmaf(__uint_as_float(r[j + 1]), sl2, -m_ref)) : 0.f;
                            lsum += p0 + p1;
                            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                            packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h);
                        }
                    }
                    const int quarter = 2 * half + (cc >> 1);
                    // the last P*V that read this quarter's previous contents is done
                    if (!(cc & 1) && p_reads[cc >> 1] > 0 && ok &&
                        !(ok = TW(2, mbar_wait(BAR(B_PEMPTY + quarter), (p_reads[cc >> 1] - 1) & 1)))) {
                        fail = ERR_SOFTMAX_P;
                    }
                    uint8_t *prow = sP + quarter * P_Q + (row >> 3) * P_SBO + (row & 7) * 16 + (cc & 1) * 4 * 128;
#pragma unroll
                    for (int kc = 0; kc < 4; ++kc)
                        *reinterpret_cast<uint4 *>(prow + kc * 128) =
                            make_uint4(packed[4 * kc], packed[4 * kc + 1], packed[4 * kc + 2], packed[4 * kc + 3]);
                    if (cc & 1) {
                        // quarter complete in this CTA once the 64 threads of this key half have written it
                        tc_fence_before_sync();
                        fence_proxy_async_smem();
                        // The first pair of quarters waits for all 128 threads: a P*V of this tile adds to every
                        // column of O, so no thread of either key half may still be rescaling its part of O.
                        if (cc == 1) named_bar_sync(1, 128);
                        else named_bar_sync(2 + half, 64);
                        if (row == 0) {
                            // (relaxed: the 64 writers have fenced their stores towards the async proxy and
                            // met at the named barrier; the arrival itself carries no data)
                            mbar_arrive_cluster_relaxed(pfull_leader + 8u * quarter);
                            if (cc == 3) mbar_arrive_cluster_relaxed(sempty_leader + 8u * b);   // this half is done with S[b]
                        }
                    }
                }
                l_run += lsum;
                const int nq = (it.n_sub - 4 * t) < 4 ? (it.n_sub - 4 * t) : 4;
                p_reads[0] += (2 * half < nq) ? 1 : 0;
                p_reads[1] += (2 * half + 1 < nq) ? 1 : 0;
            }
            if (ok && n_tiles > 0) {
                const int tl = tg0 + n_tiles - 1;
                if (!(ok = TW(3, mbar_wait(BAR(B_OREADY + (tl & 1)), (tl / 2) & 1)))) fail = ERR_SOFTMAX_END;
                tc_fence_after_sync();
            }
            tg0 += n_tiles;
            if (L == 0) { TL(3 + 3 * round); TL_ITEM(round, n_tiles); }
            TW_BEGIN(tw_epi);
            // row sum = both key halves
            named_bar_sync(1, 128);
            red[L] = l_run;
            named_bar_sync(1, 128);
            const float l_tot = l_run + red[L ^ 64];
            // ---- epilogue: thread L writes row `row`, d_v columns [256*half, 256*half + 256) ----
            const bool have = ok && n_tiles > 0 && l_tot > 0.f;
            const float inv = have ? 1.f / l_tot : 0.f;
            const bool final_out = it.final_out;
            const size_t grow = (size_t)it.g * p.R + (row_ok ? rr : 0);
            const size_t prow_idx = (size_t)it.split * p.G * p.R + grow;
            const int col0 = 256 * half;
            if (DECODE && final_out && it.rows_here == 128) {
                // bf16 result of a full decode tile (prefill measured 2 % faster with the plain row stores
                // below): staged in the (now idle) P buffer as 64-row x 64-column boxes in
                // the 128-byte swizzle and written by TMA tensor stores.  Each key-half group of 64 threads
                // (rows 0-63, 256 of the d_v columns) ping-pongs between two 8 KB boxes.
                uint8_t *box0 = sP + half * (2 * BOX);
                const int y = it.g * p.R + it.row0 + 64 * (int)rank;
#pragma unroll 1
                for (int bx = 0; bx < 4; ++bx) {
                    uint8_t *box = box0 + (bx & 1) * BOX;
                    if (bx >= 2) {
                        if (row == 0) bulk_wait_read<1>();      // the store that last read this box is done with it
                        named_bar_sync(2 + half, 64);
                    }
#pragma unroll 1
                    for (int c2 = 0; c2 < 2; ++c2) {
                        uint32_t o[32];
                        if (n_tiles > 0 && ok) {
                            tmem_ld32(tmem + lane_base + (2 * bx + c2) * 32, o);
                            tmem_wait_ld();
                        }
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
                            const int v = c2 * 4 + (j >> 3);             // 16-byte vector of the 128-byte row
                            *reinterpret_cast<uint4 *>(box + row * 128 + ((v ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    named_bar_sync(2 + half, 64);
                    if (row == 0) {
                        tma_store_2d(&tmO, col0 + 64 * bx, y, smem_u32(box));
                        bulk_commit();
                    }
                }
                if (row == 0) bulk_wait_read<0>();       // before the next item's P is written (barrier below)
            } else {
                // two 32-column reads of the accumulator in flight: the second is loaded while the first is converted and stored
                auto put = [&](const uint32_t (&o)[32], const int cc) {
                    if (!row_ok) return;
                    // 32-byte stores: a lane fills whole sectors of its own row
                    if (final_out) {
                        __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.O) + grow * p.d_v + col0 + cc * 32;
#pragma unroll
                        for (int j = 0; j < 32; j += 16) {
                            uint32_t w[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const float a = have ? __uint_as_float(o[j + 2 * e]) * inv : 0.f;
                                const float c = have ? __uint_as_float(o[j + 2 * e + 1]) * inv : 0.f;
                                __nv_bfloat162 h = __floats2bfloat162_rn(a, c);
                                w[e] = *reinterpret_cast<uint32_t *>(&h);
                            }
                            st_global_v8(dst + j, w);
                        }
                    } else {
                        float *dst = p.O_part + prow_idx * p.d_v + col0 + cc * 32;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint32_t w[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) w[e] = have ? __float_as_uint(__uint_as_float(o[j + e]) * inv) : 0u;
                            st_global_v8(dst + j, w);
                        }
                    }
                };
                const bool read_o = n_tiles > 0 && ok;
                uint32_t oa[32], ob[32];
                if (read_o) tmem_ld32(tmem + lane_base, oa);
#pragma unroll 1
                for (int cp = 0; cp < O_COLS / 64; ++cp) {
                    if (read_o) {
                        tmem_wait_ld();
                        tmem_ld32(tmem + lane_base + (2 * cp + 1) * 32, ob);
                    }
                    put(oa, 2 * cp);
                    if (read_o) {
                        tmem_wait_ld();
                        if (cp + 1 < O_COLS / 64) tmem_ld32(tmem + lane_base + (2 * cp + 2) * 32, oa);
                    }
                    put(ob, 2 * cp + 1);
                }
            }
            if (row_ok && half == 0) {
                const float m_out = have ? m_true * 0.6931471805599453f : -CUDART_INF_F;
                const float l_out = have ? l_tot * fast_exp2(m_ref - m_true) : 0.f;
                if (final_out) { p.m[grow] = m_out; p.l[grow] = l_out; }
                else { p.m_part[prow_idx] = m_out; p.l_part[prow_idx] = l_out; }
                if (it.n_parts > 0 && p.tickets == nullptr) {
                    // balanced schedule with the merge kernel: tell it which slabs of this row hold something
                    const size_t slab = (size_t)p.G * p.R;
                    if (final_out) p.l_part[grow] = -1.f;                  // "O, m, l already final"
                    else if (it.split == 0)
                        for (int sidx = it.n_parts; sidx < p.num_splits; ++sidx) {
                            p.l_part[sidx * slab + grow] = 0.f;
                            p.m_part[sidx * slab + grow] = -CUDART_INF_F;
                        }
                }
            }
            TW_END(4, tw_epi);
            TW_BEGIN(tw_merge);
            if (DECODE && it.n_parts > 1 && p.tickets != nullptr) {
                // Balanced schedule, merge in this kernel: this CTA has written its 64 rows of one piece of a cut
                // sequence.  It then draws a ticket for (sequence, CTA rank); the CTA that draws the last one finds
                // every piece of these rows in memory and merges them into O, m, l (the log-sum-exp rule of the merge
                // kernel, csrc/attention/fa2_fwd.cu:93-111 of the reference across partial results).  Nobody waits for
                // anybody.  The tickets start at zero: the launcher clears them before every launch.
                __threadfence();                                   // this thread's partial rows are visible device-wide
                named_bar_sync(1, 128);
                if (L == 0) reinterpret_cast<unsigned int *>(red)[0] = atomicAdd(&p.tickets[2 * it.g + (int)rank], 1u);
                named_bar_sync(1, 128);
                const bool last_piece = reinterpret_cast<volatile unsigned int *>(red)[0] == (unsigned)(it.n_parts - 1);
                if (last_piece) {
                    __threadfence();
                    // Each of the four warps merges 16 of the CTA's 64 rows, two rows at a time; a lane owns four
                    // consecutive d_v columns in each 128-column block, so every load and store of the warp is one
                    // contiguous run; the loads of one piece of a row pair are in flight together.
                    const size_t slab = (size_t)p.G * p.R;
                    const int np = it.n_parts < 4 ? it.n_parts : 4;        // the launcher never plans more
                    const int w4 = warp & 3;
#pragma unroll 1
                    for (int rp = 0; rp < 16; rp += 2) {
                        float wgt[2][4], mx2[2], ls2[2];
                        size_t gr[2];
                        bool okr[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int r_in = it.row0 + 64 * (int)rank + w4 * 16 + rp + e;
                            okr[e] = r_in < p.R;
                            gr[e] = (size_t)it.g * p.R + (okr[e] ? r_in : 0);
                            float lk[4], mk[4];
                            mx2[e] = -CUDART_INF_F;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                lk[k] = k < np ? __ldcg(p.l_part + k * slab + gr[e]) : 0.f;
                                mk[k] = k < np ? __ldcg(p.m_part + k * slab + gr[e]) : -CUDART_INF_F;
                                if (lk[k] > 0.f) mx2[e] = fmaxf(mx2[e], mk[k]);
                            }
                            ls2[e] = 0.f;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                wgt[e][k] = lk[k] > 0.f ? lk[k] * __expf(mk[k] - mx2[e]) : 0.f;
                                ls2[e] += wgt[e][k];
                            }
                            const float inv_l = ls2[e] > 0.f ? 1.f / ls2[e] : 0.f;
#pragma unroll
                            for (int k = 0; k < 4; ++k) wgt[e][k] *= inv_l;
                        }
                        // part by part: the eight loads of a part (two rows) are in flight together
                        float4 acc[2][4];
#pragma unroll
                        for (int e = 0; e < 2; ++e)
#pragma unroll
                            for (int j = 0; j < 4; ++j) acc[e][j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                        for (int k = 0; k < np; ++k) {
                            float4 v[2][4];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const float4 *src = reinterpret_cast<const float4 *>(p.O_part + (k * slab + gr[e]) * p.d_v) + lane;
#pragma unroll
                                for (int j = 0; j < 4; ++j) v[e][j] = __ldcg(src + 32 * j);
                            }
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const float wk = k == 0 ? wgt[e][0] : (k == 1 ? wgt[e][1] : (k == 2 ? wgt[e][2] : wgt[e][3]));
                                if (wk > 0.f) {
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        acc[e][j].x = fmaf(wk, v[e][j].x, acc[e][j].x); acc[e][j].y = fmaf(wk, v[e][j].y, acc[e][j].y);
                                        acc[e][j].z = fmaf(wk, v[e][j].z, acc[e][j].z); acc[e][j].w = fmaf(wk, v[e][j].w, acc[e][j].w);
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            if (!okr[e]) continue;
                            __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.O) + gr[e] * p.d_v + 4 * lane;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[e][j].x, acc[e][j].y), h1 = __floats2bfloat162_rn(acc[e][j].z, acc[e][j].w);
                                *reinterpret_cast<uint2 *>(dst + 128 * j) =
                                    make_uint2(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1));
                            }
                            if (lane == 0) { p.m[gr[e]] = mx2[e]; p.l[gr[e]] = ls2[e]; }
                        }
                    }
                }
            }
            TW_END(5, tw_merge);
            // this CTA's softmax warps have read O out of tensor memory: the next item may overwrite it
            // (an empty item never touched the accumulator and signals nothing)
            tc_fence_before_sync();
            named_bar_sync(1, 128);
            if (L == 0 && n_tiles > 0) mbar_arrive_cluster_relaxed(ofree_leader);
            if (L == 0) TL(4 + 3 * round);
        }
        if (L == 0) TW_FLUSH(2);
        if (!ok) atomicCAS(&g_tc_error, 0, fail ? fail : ERR_SOFTMAX);
    }

    // ---- teardown: neither CTA may leave while the pair can still touch its memory --------
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) TL(30);
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_2cta(tmem, TMEM_COLS);
    }
    if (threadIdx.x == 0) TL(31);
}

}  // namespace tc2

// --------------------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------------------

namespace tc2 {
// CTA pairs of fwd_tc2_kernel that are resident at the same time on the current device (cached per device).
static int resident_clusters() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    const int have = cached[dev].load(std::memory_order_relaxed);
    if (have > 0) return have;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaFuncSetAttribute(fwd_tc2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, fwd_tc2_kernel<true>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) return -1;
        n = sms / 2;
    }
    cached[dev].store(n, std::memory_order_relaxed);
    return n;
}
}  // namespace tc2

int fwd_tensor2_resident_clusters() { return tc2::resident_clusters(); }

bool fwd_tensor2_supported(const FwdProblem &p, int dtype) {
    if (dtype != FDMLA_BF16) return false;
    if (p.d_qk != 576 || p.d_v != 512 || p.V != nullptr) return false;
    if (p.page_table && (p.page_size % tc2::SUB) != 0) return false;
    if (p.G <= 0 || p.R <= 0 || p.num_splits <= 0) return false;
    if ((long long)((p.R + 127) / 128) * p.G * p.num_splits > 2147483647LL) return false;
    const long long kv_rows = p.page_table ? (long long)p.num_pages * p.page_size : (long long)p.G * p.Skv;
    if (kv_rows <= 0 || kv_rows > 2147483647LL || (long long)p.G * p.R > 2147483647LL) return false;
    if ((reinterpret_cast<uintptr_t>(p.Q) | reinterpret_cast<uintptr_t>(p.K)) & 15) return false;
    if ((reinterpret_cast<uintptr_t>(p.O) | reinterpret_cast<uintptr_t>(p.O_part)) & 31) return false;    // 32-byte stores
    return true;
}

int launch_fwd_tensor2(const FwdProblem &p_in, cudaStream_t stream) {
    FwdProblem p = p_in;
    // the balanced schedule is for one row tile per KV group, the whole key range and a final output
    if (p.balanced && (p.R > 128 || p.causal || p.num_splits < 2 || p.quota_min < 1 || (!p.O && p.balanced != 2) || !p.O_part ||
                       p.kv_begin > 0 || p.kv_end >= 0))
        p.balanced = 0;
    if (p.balanced == 2) { p.O = nullptr; p.tickets = nullptr; }       // balanced runs, every piece a partial
    if (!p.balanced && p.num_splits > 1) p.O = nullptr;      // equal splits: partials only
    if (!p.balanced || p.Sq != 1) p.tickets = nullptr;
    CUtensorMap tmQ, tmK, tmV, tmO;
    const long long kv_rows = p.page_table ? (long long)p.num_pages * p.page_size : (long long)p.G * p.Skv;
    if (!make_tensor_map_bf16_chunked(&tmQ, p.Q, (long long)p.G * p.R, p.d_qk, 64, 9)) return FDMLA_ERR_CUDA;
    if (!make_tensor_map_bf16_chunked(&tmV, p.K, kv_rows, p.d_qk, 64, 2)) return FDMLA_ERR_CUDA;
    if (!make_tensor_map_bf16(&tmK, p.K, kv_rows, p.d_qk, 64)) return FDMLA_ERR_CUDA;
    tmO = tmK;
    if (p.O && !make_tensor_map_bf16(&tmO, p.O, (long long)p.G * p.R, p.d_v, 64)) return FDMLA_ERR_CUDA;
    const bool decode = p.Sq == 1;
    auto kern = decode ? tc2::fwd_tc2_kernel<true> : tc2::fwd_tc2_kernel<false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2::SMEM_BYTES) != cudaSuccess)
        return FDMLA_ERR_CUDA;
    if (!decode) p.balanced = 0;
    // persistent grid: as many CTA pairs as the device keeps resident at once (one CTA per SM), each
    // walking its share of the (row tile, KV group, split) items
    const long long n_items = (long long)((p.R + 127) / 128) * p.G * p.num_splits;
    const int resident = tc2::resident_clusters();
    if (resident <= 0) return FDMLA_ERR_CUDA;
    const int n_clusters = (p.balanced || n_items >= resident) ? resident : (int)n_items;
    kern<<<dim3(2 * n_clusters), tc2::THREADS, tc2::SMEM_BYTES, stream>>>(p, tmQ, tmK, tmV, tmO);
#ifdef FDMLA_TIMELINE
    if (const char *path = getenv("FDMLA_TIMELINE_FILE")) {
        // one record per launch: n_clusters, decode flag, then the stamps and the tiles per item of every pair
        static unsigned long long stamps[tc2::TL_CLUSTERS][tc2::TL_SLOTS];
        static int tiles[tc2::TL_CLUSTERS][tc2::TL_ITEMS];
        static long long waits[tc2::TL_CLUSTERS][2][3][tc2::TW_KINDS];
        static unsigned long long tile_ts[tc2::TL_CLUSTERS][tc2::TL_TILES];
        static long long tile_clk[tc2::TL_CLUSTERS][tc2::TL_TILES];
        if (cudaStreamSynchronize(stream) == cudaSuccess &&
            cudaMemcpyFromSymbol(stamps, tc2::g_timeline, sizeof(stamps)) == cudaSuccess &&
            cudaMemcpyFromSymbol(waits, tc2::g_waits, sizeof(waits)) == cudaSuccess &&
            cudaMemcpyFromSymbol(tile_ts, tc2::g_tile_ts, sizeof(tile_ts)) == cudaSuccess &&
            cudaMemcpyFromSymbol(tile_clk, tc2::g_tile_clk, sizeof(tile_clk)) == cudaSuccess &&
            cudaMemcpyFromSymbol(tiles, tc2::g_timeline_tiles, sizeof(tiles)) == cudaSuccess) {
            if (FILE *f = fopen(path, "ab")) {
                const int head[4] = {n_clusters, decode ? 1 : 0, tc2::TL_SLOTS, tc2::TL_ITEMS};
                fwrite(head, sizeof(head), 1, f);
                fwrite(stamps, sizeof(stamps), 1, f);
                fwrite(tiles, sizeof(tiles), 1, f);
                fwrite(waits, sizeof(waits), 1, f);
                fwrite(tile_ts, sizeof(tile_ts), 1, f);
                fwrite(tile_clk, sizeof(tile_clk), 1, f);
                fclose(f);
            }
            static const unsigned long long zero[tc2::TL_CLUSTERS][tc2::TL_SLOTS] = {};
            cudaMemcpyToSymbol(tc2::g_timeline, zero, sizeof(zero));
        }
    }
#endif
    return check_launch();
}

}  // namespace fdmla
