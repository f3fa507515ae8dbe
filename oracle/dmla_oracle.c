/*
 * CPU oracle for the Flash-DMLA attention path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links or calls this file; it is the checker
 * the parity tests, the smoke test and the benchmark's CPU-baseline leg use.
 *
 * Parity status: the reference ships no golden vectors for this path.  The
 * plain-attention core of this oracle (oracle_attn_plain) is pinned against
 * outputs of the reference's own kernels (vanilla_attn_forward, fa1_forward,
 * fa2_forward) recorded on a B200 and committed under tests/golden/.  The
 * DMLA conventions layered on top (shared latent K, V = first d_v columns,
 * causal mask, paging, row statistics, backward) have no reference
 * implementation to pin against: for those parity is unpinned and the oracle
 * is cross-checked against an independent torch fp64 mirror instead.
 *
 * The arithmetic restates the reference's naive kernel
 * (csrc/attention/vanallia_attn.cu:33-82): pass 1 row max of scale*q.k
 * (:33-50), pass 2 sum of exp(s - max) (:52-69), pass 3 sum of
 * exp(s - max)/row_sum * V (:71-82).  Each dot product is computed once and
 * kept in a row buffer instead of being recomputed per output column.  Dot
 * products accumulate in fp32 in ascending k with fused multiply-add, which
 * is what nvcc makes of the reference's `dot += Qi[k] * Kj[k]`.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float dotf(const float *a, const float *b, int n)
{
    float acc = 0.f;
    for (int k = 0; k < n; ++k) acc = fmaf(a[k], b[k], acc);
    return acc;
}

/*
 * One query row against n_vis keys.  krow(j)/vrow(j) give the j-th key/value
 * row through an index array (idx == NULL means row j).  Restates
 * vanallia_attn.cu:33-82 for one block (one query row).  An empty row gives
 * m = -inf, l = 0, O = 0 (the guards of fa2_fwd.cu:99,110-111).
 */
static void attn_row(const float *q, const float *Kbase, long ldk,
                     const float *Vbase, long ldv, const long *idx, int n_vis,
                     int d_qk, int d_v, float scale, float *sbuf,
                     float *o, float *m_out, float *l_out)
{
    float row_max = -INFINITY;
    for (int j = 0; j < n_vis; ++j) {                       /* :33-50 */
        long r = idx ? idx[j] : j;
        float s = dotf(q, Kbase + r * ldk, d_qk) * scale;
        sbuf[j] = s;
        row_max = fmaxf(row_max, s);
    }
    float row_sum = 0.f;
    for (int j = 0; j < n_vis; ++j)                          /* :52-69 */
        row_sum += expf(sbuf[j] - row_max);
    for (int v = 0; v < d_v; ++v) o[v] = 0.f;
    if (n_vis > 0 && row_sum > 0.f) {
        for (int j = 0; j < n_vis; ++j) {                   /* :71-82 */
            long r = idx ? idx[j] : j;
            float p = expf(sbuf[j] - row_max) / row_sum;
            const float *vj = Vbase + r * ldv;
            for (int v = 0; v < d_v; ++v) o[v] = fmaf(p, vj[v], o[v]);
        }
    }
    *m_out = row_max;
    *l_out = row_sum;
}

/*
 * Plain single-head attention, the exact problem the reference's launchers
 * solve (vanallia_attn.cu:85-99, fa_fwd.cu:153-176, fa2_fwd.cu:139-156):
 * Q[Nq,d] K[Nk,d] V[Nk,dv] -> O[Nq,dv], non-causal.  m,l may be NULL.
 */
void oracle_attn_plain(const float *Q, const float *K, const float *V, float *O,
                       float *m, float *l, int Nq, int Nk, int d, int dv,
                       float scale)
{
    if (Nq <= 0 || Nk <= 0 || d <= 0 || dv <= 0) return;    /* :95 */
#pragma omp parallel
    {
        float *sbuf = (float *)malloc(sizeof(float) * (size_t)Nk);
#pragma omp for schedule(dynamic, 4)
        for (int i = 0; i < Nq; ++i) {
            float mm, ll;
            attn_row(Q + (size_t)i * d, K, d, V, dv, NULL, Nk, d, dv, scale,
                     sbuf, O + (size_t)i * dv, &mm, &ll);
            if (m) m[i] = mm;
            if (l) l[i] = ll;
        }
        free(sbuf);
    }
}

/* Number of keys query i sees: bottom-right aligned causal mask. */
static inline int visible(int i, int Sq, int Skv, int causal)
{
    if (!causal) return Skv;
    long n = (long)i + (long)(Skv - Sq) + 1;
    if (n < 0) n = 0;
    if (n > Skv) n = Skv;
    return (int)n;
}

/*
 * Cache-latent DMLA forward.  Q[B,H,Sq,d_qk]; K_lat[B,Skv,d_qk] shared by all
 * heads of a batch; V = K_lat[..., :d_v].  Outputs O[B,H,Sq,d_v], m,l[B,H,Sq].
 * Per row this is attn_row (vanallia_attn.cu:33-82) with the causal limit.
 */
void oracle_fwd_cache_latent(const float *Q, const float *K_lat, float *O,
                             float *m, float *l, int B, int H, int Sq, int Skv,
                             int d_qk, int d_v, float scale, int causal)
{
    long rows = (long)B * H * Sq;
#pragma omp parallel
    {
        float *sbuf = (float *)malloc(sizeof(float) * (size_t)(Skv > 0 ? Skv : 1));
#pragma omp for schedule(dynamic, 8)
        for (long r = 0; r < rows; ++r) {
            int i = (int)(r % Sq);
            int b = (int)(r / ((long)H * Sq));
            const float *Kb = K_lat + (size_t)b * Skv * d_qk;
            attn_row(Q + (size_t)r * d_qk, Kb, d_qk, Kb, d_qk, NULL,
                     visible(i, Sq, Skv, causal), d_qk, d_v, scale, sbuf,
                     O + (size_t)r * d_v, m + r, l + r);
        }
        free(sbuf);
    }
}

/* Round to the nearest bfloat16 (ties to even), returned as fp32. */
static float bf16_round(float x)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x;   /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}

/* C[M,N] = A[M,K] * B[K,N], fp32, ascending-k fused multiply-add. */
static void matmul(const float *A, const float *Bm, float *C, long M, int K, int N)
{
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        float *c = C + i * N;
        for (int n = 0; n < N; ++n) c[n] = 0.f;
        for (int k = 0; k < K; ++k) {
            float a = A[i * K + k];
            const float *b = Bm + (size_t)k * N;
            for (int n = 0; n < N; ++n) c[n] = fmaf(a, b[n], c[n]);
        }
    }
}

/*
 * On-the-fly DMLA forward.  Q[B,H,Sq,d_lat]; K,V[B,H,Skv,d_model];
 * WK,WV[d_model,d_lat] shared by every (b,h).  K_lat = K*WK, V_lat = V*WV,
 * then attn_row per query row with per-head latents, d_qk = d_v = d_lat.
 * K_lat_out / V_lat_out (may be NULL) receive the projected latents.
 * latents_bf16 != 0 rounds the projected latents to bfloat16 before the
 * attention, which is how a bf16 kernel has to store them to feed them to the
 * tensor cores.
 */
void oracle_fwd_on_the_fly(const float *Q, const float *K, const float *V,
                           const float *WK, const float *WV, float *O, float *m,
                           float *l, float *K_lat_out, float *V_lat_out, int B,
                           int H, int Sq, int Skv, int d_model, int d_lat,
                           float scale, int causal, int latents_bf16)
{
    long nkv = (long)B * H * Skv;
    float *Kl = K_lat_out ? K_lat_out : (float *)malloc(sizeof(float) * nkv * d_lat);
    float *Vl = V_lat_out ? V_lat_out : (float *)malloc(sizeof(float) * nkv * d_lat);
    matmul(K, WK, Kl, nkv, d_model, d_lat);
    matmul(V, WV, Vl, nkv, d_model, d_lat);
    if (latents_bf16)
        for (long t = 0; t < nkv * d_lat; ++t) { Kl[t] = bf16_round(Kl[t]); Vl[t] = bf16_round(Vl[t]); }
    long rows = (long)B * H * Sq;
#pragma omp parallel
    {
        float *sbuf = (float *)malloc(sizeof(float) * (size_t)(Skv > 0 ? Skv : 1));
#pragma omp for schedule(dynamic, 8)
        for (long r = 0; r < rows; ++r) {
            int i = (int)(r % Sq);
            long bh = r / Sq;
            attn_row(Q + (size_t)r * d_lat, Kl + (size_t)bh * Skv * d_lat, d_lat,
                     Vl + (size_t)bh * Skv * d_lat, d_lat, NULL,
                     visible(i, Sq, Skv, causal), d_lat, d_lat, scale, sbuf,
                     O + (size_t)r * d_lat, m + r, l + r);
        }
        free(sbuf);
    }
    if (!K_lat_out) free(Kl);
    if (!V_lat_out) free(Vl);
}

/*
 * Paged cache-latent decode (one query per sequence).  Q[B,H,d_qk];
 * kv_pool[num_pages,page_size,d_qk]; page_table[B,max_pages] maps logical page
 * -> physical page; seqlens[B].  Token t of sequence b is pool row
 * page_table[b, t / page_size] * page_size + t % page_size.  Only tokens in
 * [kv_begin, min(kv_end, seqlens[b])) are attended (kv_end < 0 means no upper
 * limit) so that a slice of the sequence yields a partial (O, m, l).
 * Outputs O[B,H,d_v], m,l[B,H].
 */
void oracle_decode_paged(const float *Q, const float *kv_pool,
                         const int32_t *page_table, const int32_t *seqlens,
                         float *O, float *m, float *l, int B, int H, int d_qk,
                         int d_v, int page_size, int max_pages, int kv_begin,
                         int kv_end, float scale)
{
#pragma omp parallel
    {
        long cap = (long)max_pages * page_size;
        long *idx = (long *)malloc(sizeof(long) * (size_t)(cap > 0 ? cap : 1));
        float *sbuf = (float *)malloc(sizeof(float) * (size_t)(cap > 0 ? cap : 1));
        long last_b = -1;
        int n = 0;
#pragma omp for schedule(dynamic, 4)
        for (long bh = 0; bh < (long)B * H; ++bh) {
            int b = (int)(bh / H);
            if (b != last_b) {              /* gather list of this sequence's pool rows */
                int hi = seqlens[b];
                if (kv_end >= 0 && kv_end < hi) hi = kv_end;
                int lo = kv_begin > 0 ? kv_begin : 0;
                n = hi > lo ? hi - lo : 0;
                for (int t = 0; t < n; ++t) {
                    int tok = lo + t;
                    idx[t] = (long)page_table[(size_t)b * max_pages + tok / page_size] *
                                 page_size + tok % page_size;
                }
                last_b = b;
            }
            size_t r = (size_t)bh;
            attn_row(Q + r * d_qk, kv_pool, d_qk, kv_pool, d_qk, idx, n, d_qk,
                     d_v, scale, sbuf, O + r * d_v, m + r, l + r);
        }
        free(idx);
        free(sbuf);
    }
}

/*
 * Merge P partial results over disjoint key sets.  O_p[P,rows,d_v] (each
 * already normalised by its own l_p), m_p,l_p[P,rows].  m = max_p m_p;
 * w_p = l_p * exp(m_p - m) (0 when l_p == 0); l = sum w_p; O = sum w_p O_p / l.
 * Same algebra as the running update of fa2_fwd.cu:93-111 (m_new, alpha,
 * l_new, beta, gamma).
 */
void oracle_merge_partials(const float *O_p, const float *m_p, const float *l_p,
                           float *O, float *m, float *l, int P, long rows,
                           int d_v)
{
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        float mx = -INFINITY;
        for (int p = 0; p < P; ++p)
            if (l_p[p * rows + r] > 0.f) mx = fmaxf(mx, m_p[p * rows + r]);
        float ls = 0.f;
        for (int p = 0; p < P; ++p) {
            float lp = l_p[p * rows + r];
            if (lp > 0.f) ls += lp * expf(m_p[p * rows + r] - mx);
        }
        float *o = O + (size_t)r * d_v;
        for (int v = 0; v < d_v; ++v) o[v] = 0.f;
        if (ls > 0.f) {
            for (int p = 0; p < P; ++p) {
                float lp = l_p[p * rows + r];
                if (!(lp > 0.f)) continue;
                float w = lp * expf(m_p[p * rows + r] - mx) / ls;
                const float *op = O_p + ((size_t)p * rows + r) * d_v;
                for (int v = 0; v < d_v; ++v) o[v] = fmaf(w, op[v], o[v]);
            }
        }
        m[r] = mx;
        l[r] = ls;
    }
}

/*
 * Tiled online-softmax forward for one head (Q[Nq,d] K[Nk,d] V[Nk,dv]), the
 * recurrence of fa2_fwd.cu:88-128: per key tile m_new = max(m_prev, m_tile),
 * alpha = exp(m_prev - m_new), l_new = l_prev*alpha + sum e, and O kept
 * normalised with beta = l_prev*alpha/l_new, gamma = 1/l_new.  Used to check
 * that the tiled algebra equals the three-pass result.
 */
void oracle_attn_online(const float *Q, const float *K, const float *V, float *O,
                        float *m, float *l, int Nq, int Nk, int d, int dv,
                        float scale, int tile)
{
    float *e = (float *)malloc(sizeof(float) * (size_t)tile);
    float *acc = (float *)malloc(sizeof(float) * (size_t)dv);
    for (int i = 0; i < Nq; ++i) {
        float m_prev = -INFINITY, l_prev = 0.f;
        float *o = O + (size_t)i * dv;
        for (int v = 0; v < dv; ++v) o[v] = 0.f;
        for (int j0 = 0; j0 < Nk; j0 += tile) {
            int cols = Nk - j0 < tile ? Nk - j0 : tile;
            float m_tile = -INFINITY;
            for (int c = 0; c < cols; ++c) {
                e[c] = dotf(Q + (size_t)i * d, K + (size_t)(j0 + c) * d, d) * scale;
                m_tile = fmaxf(m_tile, e[c]);
            }
            float m_new = fmaxf(m_prev, m_tile);
            float alpha = (m_prev == -INFINITY) ? 0.f : expf(m_prev - m_new);
            float e_sum = 0.f;
            for (int c = 0; c < cols; ++c) { e[c] = expf(e[c] - m_new); e_sum += e[c]; }
            float l_new = l_prev * alpha + e_sum;
            float beta = l_new > 0.f ? l_prev * alpha / l_new : 0.f;
            float gamma = l_new > 0.f ? 1.f / l_new : 0.f;
            for (int v = 0; v < dv; ++v) acc[v] = 0.f;
            for (int c = 0; c < cols; ++c)
                for (int v = 0; v < dv; ++v)
                    acc[v] = fmaf(e[c], V[(size_t)(j0 + c) * dv + v], acc[v]);
            for (int v = 0; v < dv; ++v) o[v] = o[v] * beta + gamma * acc[v];
            m_prev = m_new;
            l_prev = l_new;
        }
        if (m) m[i] = m_prev;
        if (l) l[i] = l_prev;
    }
    free(e);
    free(acc);
}

/*
 * Attention backward for one (batch, head) given saved row statistics.
 * Formulas of fa2_bwd.cu: delta = sum_c P*(V.dO) (:198-216) which equals
 * rowsum(dO o O); dS = P*(dP - delta) (:234); dK += dS^T Q (:252-254);
 * dV += P^T dO (:259-272); dQ += dS K (:293-309).  The reference omits the
 * softmax scale on dQ and dK; it is applied here.  P is recomputed as
 * exp(S - m) / l from the saved statistics.  dKl and dVl accumulate (caller
 * zeroes them); dQ is overwritten.
 */
static void bwd_head(const float *Q, const float *Kl, const float *Vl,
                     const float *O, const float *m, const float *l,
                     const float *dO, float *dQ, float *dKl, float *dVl, int Sq,
                     int Skv, int d_qk, int d_v, float scale, int causal)
{
    for (int i = 0; i < Sq; ++i) {
        const float *q = Q + (size_t)i * d_qk;
        const float *doi = dO + (size_t)i * d_v;
        float *dq = dQ + (size_t)i * d_qk;
        for (int k = 0; k < d_qk; ++k) dq[k] = 0.f;
        int n = visible(i, Sq, Skv, causal);
        if (n == 0 || !(l[i] > 0.f)) continue;
        float delta = dotf(doi, O + (size_t)i * d_v, d_v);
        for (int j = 0; j < n; ++j) {
            const float *kj = Kl + (size_t)j * d_qk;
            const float *vj = Vl + (size_t)j * d_v;
            float s = dotf(q, kj, d_qk) * scale;
            float p = expf(s - m[i]) / l[i];
            float dp = dotf(doi, vj, d_v);
            float ds = p * (dp - delta) * scale;
            float *dk = dKl + (size_t)j * d_qk;
            float *dv = dVl + (size_t)j * d_v;
            for (int k = 0; k < d_qk; ++k) {
                dq[k] = fmaf(ds, kj[k], dq[k]);
                dk[k] = fmaf(ds, q[k], dk[k]);
            }
            for (int v = 0; v < d_v; ++v) dv[v] = fmaf(p, doi[v], dv[v]);
        }
    }
}

/*
 * On-the-fly DMLA backward.  Inputs as oracle_fwd_on_the_fly plus O, m, l
 * (saved by the forward) and dO.  Outputs dQ[B,H,Sq,d_lat],
 * dK,dV[B,H,Skv,d_model], dWK,dWV[d_model,d_lat]:
 *   dK_lat, dV_lat per head from bwd_head; dK = dK_lat*WK^T; dV = dV_lat*WV^T;
 *   dWK = sum_{b,h} K^T dK_lat; dWV = sum_{b,h} V^T dV_lat.
 */
void oracle_bwd_on_the_fly(const float *Q, const float *K, const float *V,
                           const float *WK, const float *WV, const float *O,
                           const float *m, const float *l, const float *dO,
                           float *dQ, float *dK, float *dV, float *dWK,
                           float *dWV, int B, int H, int Sq, int Skv,
                           int d_model, int d_lat, float scale, int causal)
{
    long BH = (long)B * H;
    long nkv = BH * Skv;
    float *Kl = (float *)malloc(sizeof(float) * nkv * d_lat);
    float *Vl = (float *)malloc(sizeof(float) * nkv * d_lat);
    float *dKl = (float *)calloc((size_t)nkv * d_lat, sizeof(float));
    float *dVl = (float *)calloc((size_t)nkv * d_lat, sizeof(float));
    matmul(K, WK, Kl, nkv, d_model, d_lat);
    matmul(V, WV, Vl, nkv, d_model, d_lat);
#pragma omp parallel for schedule(dynamic, 1)
    for (long bh = 0; bh < BH; ++bh) {
        size_t qo = (size_t)bh * Sq, ko = (size_t)bh * Skv;
        bwd_head(Q + qo * d_lat, Kl + ko * d_lat, Vl + ko * d_lat, O + qo * d_lat,
                 m + qo, l + qo, dO + qo * d_lat, dQ + qo * d_lat,
                 dKl + ko * d_lat, dVl + ko * d_lat, Sq, Skv, d_lat, d_lat,
                 scale, causal);
    }
    /* dK = dK_lat * WK^T, dV = dV_lat * WV^T */
#pragma omp parallel for schedule(static)
    for (long r = 0; r < nkv; ++r) {
        for (int c = 0; c < d_model; ++c) {
            dK[r * d_model + c] = dotf(dKl + r * d_lat, WK + (size_t)c * d_lat, d_lat);
            dV[r * d_model + c] = dotf(dVl + r * d_lat, WV + (size_t)c * d_lat, d_lat);
        }
    }
    /* dWK = K^T dK_lat, dWV = V^T dV_lat, summed over every (b,h,token) in double */
#pragma omp parallel for schedule(static)
    for (int c = 0; c < d_model; ++c) {
        for (int n = 0; n < d_lat; ++n) {
            double sk = 0.0, sv = 0.0;
            for (long r = 0; r < nkv; ++r) {
                sk += (double)K[r * d_model + c] * (double)dKl[r * d_lat + n];
                sv += (double)V[r * d_model + c] * (double)dVl[r * d_lat + n];
            }
            dWK[(size_t)c * d_lat + n] = (float)sk;
            dWV[(size_t)c * d_lat + n] = (float)sv;
        }
    }
    free(Kl); free(Vl); free(dKl); free(dVl);
}

/*
 * Cache-latent backward: dQ[B,H,Sq,d_qk] and dK_lat[B,Skv,d_qk], where the
 * value gradient lands in the first d_v columns of dK_lat because
 * V = K_lat[..., :d_v].  Same per-head formulas (bwd_head); heads of a batch
 * accumulate into the shared latent.
 */
void oracle_bwd_cache_latent(const float *Q, const float *K_lat, const float *O,
                             const float *m, const float *l, const float *dO,
                             float *dQ, float *dK_lat, int B, int H, int Sq,
                             int Skv, int d_qk, int d_v, float scale, int causal)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
        const float *Kb = K_lat + (size_t)b * Skv * d_qk;
        float *dKb = dK_lat + (size_t)b * Skv * d_qk;
        float *Vl = (float *)malloc(sizeof(float) * (size_t)Skv * d_v);
        float *dVl = (float *)calloc((size_t)Skv * d_v, sizeof(float));
        for (int j = 0; j < Skv; ++j)
            memcpy(Vl + (size_t)j * d_v, Kb + (size_t)j * d_qk, sizeof(float) * d_v);
        memset(dKb, 0, sizeof(float) * (size_t)Skv * d_qk);
        for (int h = 0; h < H; ++h) {
            size_t qo = ((size_t)b * H + h) * Sq;
            bwd_head(Q + qo * d_qk, Kb, Vl, O + qo * d_v, m + qo, l + qo,
                     dO + qo * d_v, dQ + qo * d_qk, dKb, dVl, Sq, Skv, d_qk, d_v,
                     scale, causal);
        }
        for (int j = 0; j < Skv; ++j)
            for (int v = 0; v < d_v; ++v) dKb[(size_t)j * d_qk + v] += dVl[(size_t)j * d_v + v];
        free(Vl); free(dVl);
    }
}

/*
 * Balanced contiguous split of n items over `parts` ranks with the remainder
 * going to the first ranks, the rule of fa2_fwd_mpi.cu:47-53 (rows_of/off_of).
 */
void oracle_split_range(int n, int parts, int r, int *off, int *len)
{
    int base = n / parts, rem = n % parts;
    *len = base + (r < rem ? 1 : 0);
    *off = r * base + (r < rem ? r : rem);
}

/* A launcher may have pinned OpenMP to one thread (torchrun exports OMP_NUM_THREADS=1); the timed CPU
 * baseline asks for all host cores explicitly. */
void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
