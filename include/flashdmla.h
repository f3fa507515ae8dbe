/*
 * flashdmla.h - C ABI of libflashdmla.so, the B200 (sm_100a) Flash-DMLA
 * attention backend.
 *
 * Conventions shared by every entry point (they keep the style of the
 * reference's host launchers, csrc/attention/fa2_fwd.cu:139-147: raw device
 * pointers, dense row-major tensors, an explicit softmax scale, a trailing
 * stream argument):
 *   - every pointer is a DEVICE pointer owned by the caller; nothing is
 *     allocated, freed or synchronised inside the library;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) and the
 *     call returns immediately;
 *   - unlike the reference (void launchers, silent return on bad arguments:
 *     fa2_fwd.cu:149, vanallia_attn.cu:95) every call returns a status:
 *     0 on success, a negative FDMLA_ERR_* otherwise;
 *   - `dtype` selects the element type of Q/K/V/W/O/dO and gradient tensors
 *     (FDMLA_F32 or FDMLA_BF16); row statistics m, l and partial results are
 *     always fp32; accumulation is always fp32;
 *   - m[i] = max_j s_ij and l[i] = sum_j exp(s_ij - m[i]) over the visible
 *     keys of row i with s = scale * q.k (natural exp), the row_max/row_sum of
 *     vanallia_attn.cu:50,69; a row with no visible key has m=-inf, l=0, O=0;
 *   - the causal mask is bottom-right aligned: key j is visible to query i
 *     iff j <= i + (Skv - Sq).
 */
#ifndef FLASHDMLA_H_
#define FLASHDMLA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FDMLA_F32  0
#define FDMLA_BF16 1

#define FDMLA_OK               0
#define FDMLA_ERR_INVALID     -1   /* null pointer, non-positive size, bad enum      */
#define FDMLA_ERR_UNSUPPORTED -2   /* shape outside what the kernels implement        */
#define FDMLA_ERR_CUDA        -3   /* a CUDA runtime/driver call or a launch failed   */
#define FDMLA_ERR_WORKSPACE   -4   /* workspace missing or smaller than required      */
#define FDMLA_ERR_SCRATCH_LIMIT -5 /* problem exceeds the library's built-in scratch  */

/* Kernel families, for fdmla_set_backend(): AUTO picks the tcgen05/TMA kernels
 * whenever the shape qualifies and the portable CUDA-core kernels otherwise. */
#define FDMLA_BACKEND_AUTO     0
#define FDMLA_BACKEND_PORTABLE 1   /* CUDA-core kernels only (any shape)              */
#define FDMLA_BACKEND_TENSOR   2   /* tcgen05 kernels only; unsupported shapes fail   */

/* Library version (major*10000 + minor*100 + patch).  No reference counterpart. */
int fdmla_version(void);

/* Human-readable text for a status code.  No reference counterpart (the
 * reference reports no errors at all). */
const char *fdmla_status_string(int status);

/* Process-wide kernel-family override used by tests and profiling.  Replaces
 * the reference's per-call `warps_per_block` tuning knob (fa2_fwd.cu:146,150). */
int fdmla_set_backend(int backend);
int fdmla_get_backend(void);

/* on != 0 keeps the MLA-dimension shapes (576/512) on the single-CTA tcgen05
 * kernel instead of the 2-CTA cluster kernel; used for A/B measurements and to
 * keep both kernels under test.  No reference counterpart. */
int fdmla_set_single_cta(int on);

/* Name of the kernel family the last call on this thread dispatched to
 * ("tcgen05" or "portable").  No reference counterpart. */
const char *fdmla_last_kernel(void);

/* Device-side error flag of the tensor-core kernels on the current device:
 * 0 = none; 1..3, 11..17, 21..23 and 31 = a bounded wait inside a kernel gave up (which
 * kernel, role and wait; 31: a peer of fdmla_exchange_merge did not arrive); 4 = a page id outside [0, num_pages) was read from a page
 * table, or a sequence length outside [0, max_pages * page_size] was clamped.
 * Synchronises the device; reset != 0 clears the flag.  Returns -1 if the flag
 * cannot be read.
 * The flag is sticky.  After a time-out code every later tensor-core launch on
 * that device does no work at all (it writes O = 0, l = 0, m = -inf) while the
 * C call still returns FDMLA_OK, until the flag is cleared with reset != 0: a
 * caller that cannot afford silent empty results polls the flag, e.g. once per
 * step, and resets it after handling the failure.  Code 4 does not stop later
 * launches.  No reference counterpart. */
int fdmla_device_error_flag(int reset);

/*
 * Cache-latent DMLA forward.
 *   Q     [B, H, Sq, d_qk]
 *   K_lat [B, Skv, d_qk]      latent rows shared by all heads; V = K_lat[..., :d_v]
 *   O     [B, H, Sq, d_v]     m, l [B, H, Sq] fp32
 * Replaces the role of fa2_forward (csrc/attention/fa2_fwd.cu:139-156) for the
 * cache-latent mode the reference's README describes (README.md:15); per
 * (b, h) it solves the same problem as that launcher with K = K_lat[b],
 * V = K_lat[b][:, :d_v], plus the causal mask and the m/l outputs.
 */
int fdmla_fwd_cache_latent(const void *Q, const void *K_lat, void *O, float *m,
                           float *l, int B, int H, int Sq, int Skv, int d_qk,
                           int d_v, float scale, int causal, int dtype,
                           void *stream);

/*
 * On-the-fly DMLA forward: K_lat = K*WK and V_lat = V*WV are projected inside
 * the call, then attention runs on the latents.
 *   Q [B, H, Sq, d_lat]   K, V [B, H, Skv, d_model]   WK, WV [d_model, d_lat]
 *   O [B, H, Sq, d_lat]   m, l [B, H, Sq] fp32
 *   workspace: fdmla_fwd_on_the_fly_workspace_bytes() bytes of device scratch
 *   (holds the projected latents; they are left there for the backward).
 * Replaces fa2_forward (fa2_fwd.cu:139-156) for the on-the-fly mode of
 * README.md:14.
 */
size_t fdmla_fwd_on_the_fly_workspace_bytes(int B, int H, int Skv, int d_lat, int dtype);
int fdmla_fwd_on_the_fly(const void *Q, const void *K, const void *V,
                         const void *WK, const void *WV, void *O, float *m,
                         float *l, void *workspace, size_t workspace_bytes,
                         int B, int H, int Sq, int Skv, int d_model, int d_lat,
                         float scale, int causal, int dtype, void *stream);

/*
 * Paged cache-latent decode (one query token per sequence), split-KV.
 *   Q          [B, H, d_qk]
 *   kv_pool    [num_pages, page_size, d_qk]   latent rows, V = first d_v columns
 *   page_table [B, max_pages] int32           logical page -> physical page
 *   seqlens    [B] int32                      tokens held by each sequence
 *   Only tokens t with kv_begin <= t < min(kv_end, seqlens[b]) are attended
 *   (kv_end < 0: no upper limit), so a rank can compute the partial result of
 *   its slice of a long sequence.
 *   num_splits >= 1 splits the attended range of every sequence into that many
 *   page-aligned pieces computed by different thread blocks.  Their partial
 *   results go to O_part [num_splits, B, H, d_v], m_part, l_part
 *   [num_splits, B, H] (fp32, caller-provided scratch; may be NULL when
 *   num_splits == 1) and are merged into O [B, H, d_v] (dtype), m, l [B, H].
 *   If O is NULL only the partials are produced, exactly as described (piece s
 *   of every sequence in slab s).  When O is given, the scratch contents after
 *   the call are unspecified: with num_splits >= 2, the whole key range and
 *   2 <= H <= 128 the tcgen05 kernel may treat the slabs as room to cut sequences
 *   and deal the 256-key tiles of all sequences out to the SMs in equal
 *   contiguous runs; uncut sequences are written to O directly.  A cut sequence
 *   is merged either by a merge kernel (at most num_splits pieces) or, when few
 *   pieces suffice, inside the attention kernel by the thread blocks that finish
 *   its last piece (at most min(num_splits - 1, 4) pieces; the first 2 B words of
 *   the last slab of l_part then serve as arrival counters, which the call clears
 *   with a memset on `stream` before the launch).
 *   Every page id read from page_table must be in [0, num_pages) and every
 *   seqlens[b] in [0, max_pages * page_size]; a length outside is clamped and
 *   reported through fdmla_device_error_flag (code 4).
 * The paged cache is the "KV-cache" of README.md:15; per (b, h) the math is
 * that of vanilla_attn_forward (vanallia_attn.cu:85-99) on the gathered rows.
 */
int fdmla_decode_paged(const void *Q, const void *kv_pool,
                       const int32_t *page_table, const int32_t *seqlens,
                       void *O, float *m, float *l, float *O_part,
                       float *m_part, float *l_part, int B, int H, int d_qk,
                       int d_v, int page_size, int max_pages, int num_pages,
                       int num_splits, int kv_begin, int kv_end, float scale,
                       int dtype, void *stream);

/*
 * One rank's partial result of a decode whose KV sequences are split over several GPUs: attention of Q over the
 * whole of THIS cache (the rank's slice of every sequence), returned as fp32 O_out [B, H, d_v] normalised by its own
 * l_out, with m_out, l_out [B, H] - the three blocks of the message the ranks exchange and then merge with
 * fdmla_merge_lse_strided.  O_part / m_part / l_part [num_splits, ...] are private scratch (NULL for num_splits
 * == 1): the library cuts the work as it likes (on the tcgen05 path: the 256-key tiles of all sequences in equal
 * contiguous runs, which suits few long ragged sequences) and merges the pieces into the output itself.
 * With num_splits >= 2 and O_out = m_out = l_out = NULL the pieces are left unmerged in the scratch (a piece with
 * l <= 0 holds nothing) for a caller that merges them itself (fdmla_exchange_merge_parts).
 * Replaces the per-rank part of fa2_forward_mpi (csrc/attention/fa2_fwd_mpi.cu:76-90: each rank's fa2_forward over
 * its rows), for the split along the keys that long-context decode needs.
 */
int fdmla_decode_paged_partial(const void *Q, const void *kv_pool,
                               const int32_t *page_table, const int32_t *seqlens,
                               float *O_out, float *m_out, float *l_out,
                               float *O_part, float *m_part, float *l_part,
                               int B, int H, int d_qk, int d_v, int page_size,
                               int max_pages, int num_pages, int num_splits,
                               float scale, int dtype, void *stream);

/* Split count (number of scratch slabs) the library would choose for a decode
 * problem.  No reference counterpart. */
int fdmla_decode_suggest_splits(int B, int H, int max_seqlen, int d_qk, int d_v,
                                int page_size, int dtype);

/* How fdmla_decode_paged would run a problem for which a final result is wanted
 * over the whole key range: 0 = every sequence in num_splits equal pieces (or a
 * kernel other than the 2-CTA tensor kernel), 1 = balanced runs of 256-key tiles
 * with the merge kernel, 2 = balanced runs merged inside the attention kernel.
 * For 1 and 2, *quota_min receives the least number of tiles a run holds (it
 * bounds the pieces a sequence is cut into) and *units the number of runs (CTA
 * pairs resident on the current device).  A run holds
 * max(ceil(total tiles / units), quota_min) tiles.  Negative: invalid argument.
 * No reference counterpart. */
int fdmla_decode_plan(int B, int H, int d_qk, int d_v, int page_size,
                      int max_pages, int num_splits, int dtype, int *quota_min,
                      int *units);

/*
 * fdmla_decode_paged for callers that cannot allocate device memory.  It has no counterpart
 * in the reference.  Same computation and same arguments as fdmla_decode_paged over the
 * whole sequence (kv_begin = 0, no kv_end), but the split-KV partials are kept in a 32 MiB
 * array that is part of the library image, so the caller passes no scratch buffers and the
 * call itself never allocates or frees anything.  It is meant for code that runs where an
 * allocation is impossible or forbidden: after all device memory has been handed to a pool
 * the caller does not own, inside hosts that do not let an operator call the allocator, or
 * on a latency path where an allocation would synchronise the device.
 *   - The final O, m, l are always produced (O must not be NULL).
 *   - num_splits * B * H must not exceed fdmla_decode_paged_noalloc_max_rows(d_v)
 *     (16 320 rows at d_v = 512); a larger problem is refused with
 *     FDMLA_ERR_SCRATCH_LIMIT and nothing is launched.  num_splits == 1 needs no scratch.
 *   - The first call on a device looks up the array's device address; make that first call
 *     outside any stream capture.
 *   - Every call on a device shares the one array and it keeps the previous call's contents.
 *     The caller clears nothing (each call overwrites every slot it later reads and zeroes the
 *     few counters that must start at zero with a memset on `stream`), but
 *     two calls that overlap on the GPU (different streams, or different host threads) race
 *     on it: serialise them, or use fdmla_decode_paged with separate buffers.
 *   - Each GPU that loads the library holds the 32 MiB until the process exits.
 */
size_t fdmla_decode_paged_noalloc_max_rows(int d_v);
int fdmla_decode_paged_noalloc(const void *Q, const void *kv_pool,
                               const int32_t *page_table, const int32_t *seqlens,
                               void *O, float *m, float *l, int B, int H, int d_qk,
                               int d_v, int page_size, int max_pages, int num_pages,
                               int num_splits, float scale, int dtype, void *stream);

/*
 * Log-sum-exp merge of partial attention results over disjoint key sets.
 *   O_part [num_parts, rows, d_v] fp32 (each normalised by its own l_part)
 *   m_part, l_part [num_parts, rows] fp32
 *   O [rows, d_v] (out_dtype), m, l [rows] fp32
 * m = max_p m_p; w_p = l_p exp(m_p - m); l = sum w_p; O = sum w_p O_p / l:
 * the running update of fa2_fwd.cu:93-111 applied across partials.
 */
int fdmla_merge_lse(const float *O_part, const float *m_part,
                    const float *l_part, void *O, float *m, float *l,
                    long long rows, int d_v, int num_parts, int out_dtype,
                    void *stream);

/* The same merge over partials that are not stored back to back: part p of
 * O_part starts part_stride_o floats after part p - 1 (>= rows * d_v), part p of
 * m_part / l_part part_stride_ml floats after part p - 1 (>= rows).  This is the
 * layout of all-gathered messages that each hold one rank's O, m and l one after
 * the other (the exchange step that replaces the host all-gather of
 * csrc/attention/fa2_fwd_mpi.cu:65-74). */
int fdmla_merge_lse_strided(const float *O_part, const float *m_part,
                            const float *l_part, void *O, float *m, float *l,
                            long long rows, int d_v, int num_parts,
                            long long part_stride_o, long long part_stride_ml,
                            int out_dtype, void *stream);

/*
 * Exchange and merge of the ranks' partial results in one kernel over peer memory (NVLink), for the GPUs of one
 * node, one process per GPU: the fused form of "all-gather the messages, then fdmla_merge_lse_strided".
 * It replaces the same exchange step as the all-gather does (the host MPI_Allgatherv of
 * csrc/attention/fa2_fwd_mpi.cu:65-74) with the merge rule of fa2_fwd.cu:93-111; the reference has no device-side
 * exchange.
 *
 * Set-up, once per (world, rows, d_v): every rank allocates an exchange buffer of fdmla_exchange_bytes with
 * fdmla_exchange_alloc (device memory, zeroed; ipc_handle receives 64 bytes that name it to other processes),
 * hands the handle to its peers by any host channel, maps every peer's buffer with fdmla_exchange_open, and
 * synchronises with its peers on the host once before the first step.  fdmla_exchange_close unmaps a peer's
 * buffer, fdmla_exchange_free releases the rank's own.
 *
 * A step, on every rank: msg is the rank's message [ O (rows x d_v) | m (rows) | l (rows) ] fp32 (what
 * fdmla_decode_paged_partial writes); bufs[p], p < world, is rank p's buffer as mapped in this process
 * (bufs[rank] the rank's own; a host array).  Up to four ranks, the kernel stores the whole message into every
 * peer's buffer, waits for the peers' and merges everything itself (one NVLink hop).  Beyond four, the rows are
 * dealt to the ranks in 128 runs; the kernel stores its partial rows of a run into the buffer of the rank that
 * owns the run, and for the runs it owns itself waits for its peers' rows, merges, and stores the merged rows
 * into every peer's buffer, from where each copies them out (two hops; a rank sends (world - 1) / world of a
 * message and its share of the results).  Either way every rank ends with the merged O [rows, d_v] (out_dtype),
 * m, l [rows].  The arithmetic is that of fdmla_merge_lse_strided on the all-gathered
 * messages, part by part in rank order (bit-identical to it up to 4096 rows, where that merge sums in the same
 * order).  FDMLA_EXCHANGE_GATHER=1 / 0 in the environment (of every rank alike) forces the first / second form.
 * All ranks must issue the same sequence of steps on one set of buffers, each rank from one stream (a step may
 * be captured into a CUDA graph: the step counter lives in the buffer).  A peer that does not arrive
 * within timeout_ms leaves O, m, l of the affected rows unwritten and sets fdmla_device_error_flag code 31; the
 * buffers must then be set up again.
 * world <= 16, d_v a multiple of 4.
 */
size_t fdmla_exchange_bytes(int world, long long rows, int d_v);
int fdmla_exchange_alloc(size_t bytes, void **buf, void *ipc_handle);
int fdmla_exchange_open(const void *ipc_handle, void **peer_buf);
int fdmla_exchange_close(void *peer_buf);
int fdmla_exchange_free(void *buf);
int fdmla_exchange_merge(const float *msg, void *const *bufs, int world, int rank,
                         long long rows, int d_v, void *O, float *m, float *l,
                         int out_dtype, int timeout_ms, void *stream);
/* The same step when the rank's own partial result is still in num_parts (1..64) pieces - O_part [num_parts, rows,
 * d_v], m_part, l_part [num_parts, rows] fp32, dense, pieces with l <= 0 hold nothing: what
 * fdmla_decode_paged_partial leaves in its scratch when it is called without outputs.  The kernel first merges the
 * pieces into msg (written, then sent), so the local merge, the exchange and the final merge are one launch. */
int fdmla_exchange_merge_parts(const float *O_part, const float *m_part,
                               const float *l_part, int num_parts, float *msg,
                               void *const *bufs, int world, int rank, long long rows,
                               int d_v, void *O, float *m, float *l, int out_dtype,
                               int timeout_ms, void *stream);

/*
 * Batched bf16 GEMM on the tensor cores, fp32 accumulation: C[b] (M x N) = A[b] (M x K) * B[b] for b < batch.
 * It serves the GEMMs either side of the attention kernel that the reference's README.md:16-20 describes and
 * ships no source for: the "absorbed" query and output projections of an MLA block (batch = heads) and the
 * expert MLPs of the MoE layer over padded packing (batch = experts).
 *   Every operand is a window of a 2-D row-major bf16 tensor with `ld*` elements per row: batch entry b of A
 *   starts at row b * a_brow and column b * a_bcol of a tensor of a_rows rows, so that a batch may run down the
 *   rows (experts) or across the columns (heads of a [tokens, heads * width] activation); B and C likewise.
 *   b_k_major != 0: B's tensor holds [N, K] windows (rows = output columns, the reduction index contiguous);
 *   b_k_major == 0: [K, N] windows (rows = reduction index, the output column contiguous).
 *   gated != 0: C = silu(A * B) .* (A * B2) (the SwiGLU gate of an expert MLP in the GEMM's epilogue); B2 has
 *   B's geometry.  B2 is ignored otherwise and may be NULL.
 *   Limits: K % 64 == 0, N % 64 == 0 (gated: % 128), lda % 8 == 0, ldb % 64 == 0, ldc % 16 == 0, a_bcol % 8 == 0,
 *   b_bcol % 64 == 0, c_bcol % 16 == 0, A, B 16-byte and C 32-byte aligned; FDMLA_ERR_UNSUPPORTED otherwise, and
 *   when the kernel family is forced to the portable one (there is no CUDA-core GEMM in this library).
 *   Windows that do not fit their tensors are refused (FDMLA_ERR_INVALID).
 */
int fdmla_gemm_batched(const void *A, const void *B, const void *B2, void *C,
                       int batch, int M, int N, int K, long long a_rows,
                       long long lda, int a_brow, int a_bcol, long long b_rows,
                       long long ldb, int b_brow, int b_bcol, int b_k_major,
                       long long ldc, long long c_brow, long long c_bcol,
                       int gated, void *stream);

/*
 * The same GEMM over groups of rows whose sizes only the device knows: group g owns rows
 * [row_offsets[g], row_offsets[g + 1]) of A [total_rows, lda] and of C [total_rows, ldc] (row_offsets: groups + 1
 * int32 in device memory, ascending, row_offsets[groups] <= total_rows) and multiplies them with its own window of B
 * (rows g * b_brow ... of a tensor of b_rows rows; K-major or MN-major as above).  This is the expert MLP over the
 * packed rows of fdmla_moe_pack without padding and without reading the counts back to the host (the "grouped GEMM"
 * of the reference's advertised csrc/moe, README.md:19,48-53; no source there).  gated as above.
 */
int fdmla_gemm_grouped(const void *A, const void *B, const void *B2, void *C,
                       const int32_t *row_offsets, int groups, int total_rows,
                       int N, int K, long long lda, long long b_rows,
                       long long ldb, int b_brow, int b_k_major, long long ldc,
                       int gated, void *stream);

/*
 * Rotary embedding of `rows` bf16 rows of width d that sit inside wider tensors (row strides ldx, ldy elements):
 * y[r, 2i], y[r, 2i+1] = rotation of x[r, 2i], x[r, 2i+1] by the angle pos[r / rows_per_pos] * base^(-2i/d).
 * The RoPE tail of the absorbed query: read from the per-head query, written next to the 512 latent columns
 * that fdmla_gemm_batched produced (README.md:16; no source in the reference).
 */
int fdmla_rope_rows(const void *x, long long ldx, void *y, long long ldy,
                    const int32_t *pos, long long rows, int rows_per_pos, int d,
                    float base, void *stream);

/*
 * On-the-fly DMLA backward.  Inputs of the forward plus its outputs O, m, l
 * and the incoming gradient dO [B, H, Sq, d_lat].  P is recomputed from the
 * saved m, l.  Outputs (overwritten, no pre-zeroing needed, no atomics):
 *   dQ [B, H, Sq, d_lat]   dK, dV [B, H, Skv, d_model]   dWK, dWV [d_model, d_lat]
 *   workspace: fdmla_bwd_on_the_fly_workspace_bytes() bytes of device scratch.
 * Replaces fa2_backward (csrc/attention/fa2_bwd.cu:332-356), whose formulas
 * (:198-216, :234, :252-254, :259-272, :293-309) it follows with the softmax
 * scale applied to dQ and dK_lat.
 */
size_t fdmla_bwd_on_the_fly_workspace_bytes(int B, int H, int Sq, int Skv,
                                            int d_model, int d_lat, int dtype);
int fdmla_bwd_on_the_fly(const void *Q, const void *K, const void *V,
                         const void *WK, const void *WV, const void *O,
                         const float *m, const float *l, const void *dO,
                         void *dQ, void *dK, void *dV, void *dWK, void *dWV,
                         void *workspace, size_t workspace_bytes, int B, int H,
                         int Sq, int Skv, int d_model, int d_lat, float scale,
                         int causal, int dtype, void *stream);

/*
 * Cache-latent backward: dQ [B, H, Sq, d_qk] and dK_lat [B, Skv, d_qk]; the
 * value gradient is folded into the first d_v columns of dK_lat because
 * V = K_lat[..., :d_v].  Same formulas as above (fa2_bwd.cu:198-309).
 *   workspace: fdmla_bwd_cache_latent_workspace_bytes() bytes.  bf16 problems whose d_qk, d_v and Skv are multiples
 *   of 64 run as tensor-core GEMMs with the score matrices of up to 131 072 query rows at a time in the workspace
 *   (at most about 2 GB beside B*H*Sq floats and up to 16 fp32 copies of a batch entry's dK_lat); everything else runs
 *   on the CUDA-core kernels and needs B*H*Sq floats.
 */
size_t fdmla_bwd_cache_latent_workspace_bytes(int B, int H, int Sq, int Skv,
                                              int d_qk, int d_v, int dtype);
int fdmla_bwd_cache_latent(const void *Q, const void *K_lat, const void *O,
                           const float *m, const float *l, const void *dO,
                           void *dQ, void *dK_lat, void *workspace,
                           size_t workspace_bytes, int B, int H, int Sq,
                           int Skv, int d_qk, int d_v, float scale, int causal,
                           int dtype, void *stream);

/*
 * Copy `n_tokens` new latent rows per sequence into the paged pool.
 *   new_rows [B, n_tokens, d_qk]; token t of sequence b is written at logical
 *   position start_pos[b] + t through page_table.
 * The writer side of the cache the decode consumes (README.md:15); no source
 * for it exists in the reference.
 */
int fdmla_cache_append(const void *new_rows, void *kv_pool,
                       const int32_t *page_table, const int32_t *start_pos,
                       int B, int n_tokens, int d_qk, int page_size,
                       int max_pages, int num_pages, int dtype, void *stream);

/*
 * Gather the first n_tokens logical rows of every sequence into a dense
 * [B, n_tokens, d_qk] tensor (rows past seqlens[b] are zero).  Used to check
 * page-table indexing bit-exactly.  No reference counterpart.
 */
int fdmla_cache_gather(const void *kv_pool, const int32_t *page_table,
                       const int32_t *seqlens, void *out, int B, int n_tokens,
                       int d_qk, int page_size, int max_pages, int num_pages,
                       int dtype, void *stream);

/* --------------------------------------------------------------------------
 * MoE FFN plumbing (the "unfused reference path" of README.md:17-20: Top-K gate
 * -> per-expert packing (bucket + exclusive scan) -> expert MLP -> combine and
 * shared-expert add; the reference lists csrc/moe/router_topk.cu,
 * pack_dispatch.cu, combine_scatter.cu at README.md:48-53 but ships none).
 * The expert MLPs themselves are two grouped GEMMs: fdmla_gemm_batched above with
 * the experts as the batch (the first one with the SwiGLU gate in its epilogue);
 * the calls below are what surrounds them.
 * -------------------------------------------------------------------------- */

/*
 * Gate.  logits [T, E] fp32.  p = softmax(logits); the k largest win (ties:
 * lower expert index), listed by descending p; w = p / sum of the selected p.
 *   idx [T, k] int32, w [T, k] fp32.  k <= 32, E <= 2048.
 */
int fdmla_moe_route_topk(const float *logits, int32_t *idx, float *w, int T,
                         int E, int k, void *stream);

/*
 * Packing.  Assignment a = t * k + j goes to expert idx[a]; inside an expert
 * the assignments keep their order; an expert keeps its first `capacity`
 * assignments and drops the rest.
 *   offsets [E + 1]: exclusive scan of the kept counts (offsets[E] = packed rows)
 *   pos     [T, k]:  packed row of every assignment, -1 if dropped
 *   perm    [>= min(T k, E capacity)]: token of every packed row
 * Deterministic (no atomics decide an order).  Workspace: see below.
 * padded != 0: every expert owns `capacity` rows (offsets[e] = e * capacity),
 * so that the packed rows form an [E, capacity, d] batch for a batched GEMM;
 * rows past an expert's count hold nothing and no assignment points at them
 * (perm then has E * capacity entries, those of unused rows are -1 and
 * fdmla_moe_gather writes zeros for them).
 */
size_t fdmla_moe_pack_workspace_bytes(int T, int k, int E);
int fdmla_moe_pack(const int32_t *idx, int32_t *pos, int32_t *perm,
                   int32_t *offsets, void *workspace, size_t workspace_bytes,
                   int T, int k, int E, int capacity, int padded, void *stream);

/*
 * packed[r, :] = x[perm[r], :] for r < offsets[E] (read on the device);
 * max_rows only sizes the launch.  Rows of d elements, d * elem size a
 * multiple of 16 bytes.
 */
int fdmla_moe_gather(const void *x, const int32_t *perm, const int32_t *offsets,
                     void *packed, int max_rows, int E, int d, int dtype,
                     void *stream);

/*
 * The same packed rows written from the token side: packed[pos[t, j], :] =
 * x[t, :] for every kept assignment.  Every token row is read once (the
 * gather reads it once per assignment).  k <= 32.
 */
int fdmla_moe_scatter(const void *x, const int32_t *pos, void *packed, int T,
                      int k, int d, int dtype, void *stream);

/*
 * out[t, :] = sum_j w'[t, j] * y[pos[t, j], :] (+ shared[t, :] if not NULL),
 * w' = the weights of the kept assignments rescaled to sum to 1 ("gate weight
 * renormalization under capacity; overflow tokens are masked", README.md:20).
 * fp32 accumulation; y, shared, out in `dtype`.
 */
int fdmla_moe_combine(const void *y, const int32_t *pos, const float *w,
                      const void *shared, void *out, int T, int k, int d,
                      int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHDMLA_H_ */
