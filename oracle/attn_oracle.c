/*
 * attn_oracle.c -- CPU restatement (fp64 arithmetic) of Sentinel's causal
 * self-attention core, forward and backward.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the CUDA path is
 * compared against; nothing in the shipped library links, loads or calls it.
 *
 * What it restates (paths are relative to the reference project root):
 *   forward   sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:232-254
 *             per query head: scores[key][query] = scale * K^T Q, forbidden
 *             (key > query) entries masked, softmax over keys, O = V * P
 *             (computeDenseMaskedScoresInto :122-126, Softmax.cpp:10-44,
 *             attendDenseInto :150-152)
 *   GQA       kvHead = queryHead / (Hq / Hkv)     (:90-93)
 *   backward  sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:333-352
 *             dV = dO * P^T ; dP = V^T * dO ; dS = P o (dP - sum_k dP o P)
 *             (softmaxBackwardInto :194-210); forbidden dS zeroed; dS *= scale;
 *             dQ = K * dS ; dK = Q * dS^T ; dK/dV summed over the query heads
 *             of a group (addHeadInto :351-352)
 *   LSE       sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:1258-1265
 *             lse = m + ln(sum_k exp(s_k - m)), natural log, per (head, query)
 *   Delta     sentinel/NeuralNet/Cuda/CudaFlashAttention.cu:576-596
 *             delta = rowsum(dO o O)  (equals sum_k dP o P)
 *
 * Parity pin: checked against outputs of the reference's own CPU layer
 * (compiled from the reference sources into oracle/_ref, driven through its
 * public API) that are committed as fixtures under tests/golden/.
 *
 * Tensor layout of this file: token-major [B][H][S][D] ("BHSD"), fp32 in
 * memory, element (b,h,s,d) at ((b*H + h)*S + s)*D + d.  All arithmetic is
 * double; results are rounded to fp32 once when stored.  LSE is [B][Hq][Sq].
 *
 * Sequence lengths may differ between queries and keys (used by the ring
 * schedule's off-diagonal blocks, which are non-causal).  With causal != 0 a
 * key j is visible to query i iff j <= i + (Skv - Sq): query i sits at
 * position i + (Skv - Sq), the case of new tokens attending a KV cache
 * (sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:318-341); the window is
 * measured from that position too.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

typedef struct {
    int batch, q_heads, kv_heads, seq_q, seq_kv, head_dim, causal;
    float scale;
    int window;        /* sliding window (keys a query sees counting itself); <= 0: unlimited; needs causal */
    int global_tokens; /* the first global_tokens keys stay visible to every later query */
} oracle_shape;

/* The window part of CausalSelfAttention::allowsKey (sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:95-100):
 * below the causal limit a key is visible iff it is a global token, or there is no window, or it lies inside
 * [query - window + 1, query]. */
static inline int window_allows(const oracle_shape* s, int query, int key)
{
    if (!s->causal || s->window <= 0) return 1;
    if (key < s->global_tokens) return 1;
    return key >= query - s->window + 1;
}

static inline int visible_keys(const oracle_shape* s, int query)
{
    if (!s->causal) return s->seq_kv;
    long limit = (long)query + (long)(s->seq_kv - s->seq_q) + 1;
    if (limit < 0) limit = 0;
    if (limit > s->seq_kv) limit = s->seq_kv;
    return (int)limit;
}

/* scores of query row `query` against keys [0, n): returns max; p[] receives raw scores, -inf for keys the window
 * hides (they then get probability exactly 0 everywhere downstream) */
static double score_row(const oracle_shape* s, int query, const float* q, const float* kbase, int n, int d, double scale,
                        double* p)
{
    double m = -INFINITY;
    for (int j = 0; j < n; ++j) {
        if (!window_allows(s, query + (s->causal ? s->seq_kv - s->seq_q : 0), j)) { p[j] = -INFINITY; continue; }
        const float* k = kbase + (size_t)j * d;
        double acc = 0.0;
        for (int t = 0; t < d; ++t) acc += (double)q[t] * (double)k[t];
        acc *= scale;
        p[j] = acc;
        if (acc > m) m = acc;
    }
    return m;
}

/*
 * Forward.  q:[B][Hq][Sq][D]  k,v:[B][Hkv][Skv][D]  ->  o:[B][Hq][Sq][D], lse:[B][Hq][Sq].
 * A query row with no visible key gets O = 0 and LSE = -inf.
 */
int oracle_attn_fwd(const oracle_shape* s, const float* q, const float* k, const float* v,
                    float* o, float* lse)
{
    if (!s || s->q_heads % s->kv_heads != 0) return 1;
    const int D = s->head_dim, group = s->q_heads / s->kv_heads;
    const long rows = (long)s->batch * s->q_heads * s->seq_q;
#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)(s->seq_kv > 0 ? s->seq_kv : 1));
        double* acc = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(dynamic, 16)
        for (long r = 0; r < rows; ++r) {
            const int i = (int)(r % s->seq_q);
            const int h = (int)((r / s->seq_q) % s->q_heads);
            const int b = (int)(r / ((long)s->seq_q * s->q_heads));
            const int hk = h / group;
            const float* qrow = q + (size_t)r * D;
            const float* kb = k + ((size_t)b * s->kv_heads + hk) * (size_t)s->seq_kv * D;
            const float* vb = v + ((size_t)b * s->kv_heads + hk) * (size_t)s->seq_kv * D;
            const int n = visible_keys(s, i);
            for (int t = 0; t < D; ++t) acc[t] = 0.0;
            if (n == 0) {
                for (int t = 0; t < D; ++t) o[(size_t)r * D + t] = 0.0f;
                lse[r] = -INFINITY;
                continue;
            }
            const double m = score_row(s, i, qrow, kb, n, D, (double)s->scale, p);
            double l = 0.0;
            for (int j = 0; j < n; ++j) { p[j] = exp(p[j] - m); l += p[j]; }
            for (int j = 0; j < n; ++j) {
                const double w = p[j] / l;
                const float* vr = vb + (size_t)j * D;
                for (int t = 0; t < D; ++t) acc[t] += w * (double)vr[t];
            }
            for (int t = 0; t < D; ++t) o[(size_t)r * D + t] = (float)acc[t];
            lse[r] = (float)(m + log(l));
        }
        free(p);
        free(acc);
    }
    return 0;
}

/*
 * Backward.  Recomputes P from scratch in fp64 (it does not consume an LSE, so
 * it is independent of the forward under test).  dq:[B][Hq][Sq][D], dk,dv:
 * [B][Hkv][Skv][D]; all three are overwritten.  delta (optional, may be NULL)
 * receives rowsum(dO o O) as [B][Hq][Sq].
 */
int oracle_attn_bwd(const oracle_shape* s, const float* q, const float* k, const float* v,
                    const float* dout, float* dq, float* dk, float* dv, float* delta)
{
    if (!s || s->q_heads % s->kv_heads != 0) return 1;
    const int D = s->head_dim, group = s->q_heads / s->kv_heads;
    const size_t kv_elems = (size_t)s->batch * s->kv_heads * s->seq_kv * D;
    const long kv_slabs = (long)s->batch * s->kv_heads;

    /* parallel over (batch, kv head): each slab owns its dK/dV, so no races and a fixed summation order */
    double* dk_acc = (double*)calloc(kv_elems ? kv_elems : 1, sizeof(double));
    double* dv_acc = (double*)calloc(kv_elems ? kv_elems : 1, sizeof(double));
    if (!dk_acc || !dv_acc) { free(dk_acc); free(dv_acc); return 2; }

#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)(s->seq_kv > 0 ? s->seq_kv : 1));
        double* dp = (double*)malloc(sizeof(double) * (size_t)(s->seq_kv > 0 ? s->seq_kv : 1));
        double* dq_acc = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(dynamic, 1)
        for (long slab = 0; slab < kv_slabs; ++slab) {
            const int b = (int)(slab / s->kv_heads), hk = (int)(slab % s->kv_heads);
            const float* kb = k + (size_t)slab * s->seq_kv * D;
            const float* vb = v + (size_t)slab * s->seq_kv * D;
            double* dkb = dk_acc + (size_t)slab * s->seq_kv * D;
            double* dvb = dv_acc + (size_t)slab * s->seq_kv * D;
            for (int g = 0; g < group; ++g) {
                const int h = hk * group + g;
                for (int i = 0; i < s->seq_q; ++i) {
                    const size_t r = ((size_t)b * s->q_heads + h) * s->seq_q + i;
                    const float* qrow = q + r * D;
                    const float* dorow = dout + r * D;
                    const int n = visible_keys(s, i);
                    for (int t = 0; t < D; ++t) dq_acc[t] = 0.0;
                    double dl = 0.0;
                    if (n > 0) {
                        const double m = score_row(s, i, qrow, kb, n, D, (double)s->scale, p);
                        double l = 0.0;
                        for (int j = 0; j < n; ++j) { p[j] = exp(p[j] - m); l += p[j]; }
                        for (int j = 0; j < n; ++j) {
                            p[j] /= l;
                            const float* vr = vb + (size_t)j * D;
                            double a = 0.0;
                            for (int t = 0; t < D; ++t) a += (double)vr[t] * (double)dorow[t];
                            dp[j] = a;
                            dl += a * p[j];
                        }
                        for (int j = 0; j < n; ++j) {
                            const double ds = p[j] * (dp[j] - dl) * (double)s->scale;
                            const float* kr = kb + (size_t)j * D;
                            double* dkr = dkb + (size_t)j * D;
                            double* dvr = dvb + (size_t)j * D;
                            for (int t = 0; t < D; ++t) {
                                dq_acc[t] += ds * (double)kr[t];
                                dkr[t] += ds * (double)qrow[t];
                                dvr[t] += p[j] * (double)dorow[t];
                            }
                        }
                    }
                    for (int t = 0; t < D; ++t) dq[r * D + t] = (float)dq_acc[t];
                    if (delta) delta[r] = (float)dl;
                }
            }
        }
        free(p);
        free(dp);
        free(dq_acc);
    }
    for (size_t e = 0; e < kv_elems; ++e) { dk[e] = (float)dk_acc[e]; dv[e] = (float)dv_acc[e]; }
    free(dk_acc);
    free(dv_acc);
    return 0;
}

/*
 * Sampled oracle for long sequences: forward rows and dQ rows for a list of
 * query indices of one (b, h).  o_rows/dq_rows: [n_rows][D]; lse_rows: [n_rows].
 * dq_rows may be NULL (forward only); dout is then unused.
 */
int oracle_attn_rows(const oracle_shape* s, int b, int h, const float* q, const float* k, const float* v,
                     const float* dout, const int* rows, int n_rows, float* o_rows, float* lse_rows,
                     float* dq_rows)
{
    if (!s || s->q_heads % s->kv_heads != 0) return 1;
    const int D = s->head_dim, group = s->q_heads / s->kv_heads, hk = h / group;
    const float* kb = k + ((size_t)b * s->kv_heads + hk) * (size_t)s->seq_kv * D;
    const float* vb = v + ((size_t)b * s->kv_heads + hk) * (size_t)s->seq_kv * D;
#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)(s->seq_kv > 0 ? s->seq_kv : 1));
        double* acc = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(dynamic, 1)
        for (int x = 0; x < n_rows; ++x) {
            const int i = rows[x];
            const size_t r = ((size_t)b * s->q_heads + h) * s->seq_q + i;
            const float* qrow = q + r * D;
            const int n = visible_keys(s, i);
            for (int t = 0; t < D; ++t) acc[t] = 0.0;
            if (n == 0) {
                for (int t = 0; t < D; ++t) { o_rows[(size_t)x * D + t] = 0.0f; if (dq_rows) dq_rows[(size_t)x * D + t] = 0.0f; }
                lse_rows[x] = -INFINITY;
                continue;
            }
            const double m = score_row(s, i, qrow, kb, n, D, (double)s->scale, p);
            double l = 0.0;
            for (int j = 0; j < n; ++j) { p[j] = exp(p[j] - m); l += p[j]; }
            for (int j = 0; j < n; ++j) {
                p[j] /= l;
                const float* vr = vb + (size_t)j * D;
                for (int t = 0; t < D; ++t) acc[t] += p[j] * (double)vr[t];
            }
            for (int t = 0; t < D; ++t) o_rows[(size_t)x * D + t] = (float)acc[t];
            lse_rows[x] = (float)(m + log(l));
            if (dq_rows) {
                const float* dorow = dout + r * D;
                double dl = 0.0;
                for (int t = 0; t < D; ++t) dl += acc[t] * (double)dorow[t];
                for (int t = 0; t < D; ++t) acc[t] = 0.0;
                for (int j = 0; j < n; ++j) {
                    const float* vr = vb + (size_t)j * D;
                    const float* kr = kb + (size_t)j * D;
                    double a = 0.0;
                    for (int t = 0; t < D; ++t) a += (double)vr[t] * (double)dorow[t];
                    const double ds = p[j] * (a - dl) * (double)s->scale;
                    for (int t = 0; t < D; ++t) acc[t] += ds * (double)kr[t];
                }
                for (int t = 0; t < D; ++t) dq_rows[(size_t)x * D + t] = (float)acc[t];
            }
        }
        free(p);
        free(acc);
    }
    return 0;
}

/*
 * Sampled oracle, key side: dK and dV rows for a list of key indices of one
 * (b, kv head).  Needs every query of the group that can see the key, so cost is
 * O(group * Sq * Skv * D) per call regardless of n_cols: it recomputes each query
 * row's softmax statistics once and then touches only the sampled keys.
 * dk_rows, dv_rows: [n_cols][D].
 */
int oracle_attn_cols(const oracle_shape* s, int b, int hk, const float* q, const float* k, const float* v,
                     const float* dout, const int* cols, int n_cols, float* dk_rows, float* dv_rows)
{
    if (!s || s->q_heads % s->kv_heads != 0) return 1;
    const int D = s->head_dim, group = s->q_heads / s->kv_heads;
    const float* kb = k + ((size_t)b * s->kv_heads + hk) * (size_t)s->seq_kv * D;
    const float* vb = v + ((size_t)b * s->kv_heads + hk) * (size_t)s->seq_kv * D;
    const long n_q = (long)group * s->seq_q;
    int min_col = s->seq_kv;
    for (int c = 0; c < n_cols; ++c) if (cols[c] < min_col) min_col = cols[c];
    int threads = 1;
#if defined(_OPENMP)
    threads = omp_get_max_threads();
#endif
    const size_t slab = (size_t)n_cols * D;
    double* dk_part = (double*)calloc((size_t)threads * slab * 2 + 1, sizeof(double));
    if (!dk_part) return 2;
#pragma omp parallel
    {
        int tid = 0;
#if defined(_OPENMP)
        tid = omp_get_thread_num();
#endif
        double* dk_acc = dk_part + (size_t)tid * slab * 2;
        double* dv_acc = dk_acc + slab;
        double* p = (double*)malloc(sizeof(double) * (size_t)(s->seq_kv > 0 ? s->seq_kv : 1));
#pragma omp for schedule(dynamic, 8)
        for (long x = 0; x < n_q; ++x) {
            const int g = (int)(x / s->seq_q), i = (int)(x % s->seq_q);
            const int h = hk * group + g;
            const size_t r = ((size_t)b * s->q_heads + h) * s->seq_q + i;
            const float* qrow = q + r * D;
            const float* dorow = dout + r * D;
            const int n = visible_keys(s, i);
            if (n == 0 || n <= min_col) continue;      /* this query sees none of the sampled keys */
            int any = 0;                               /* a query whose dO row is all zero adds nothing to dK, dV */
            for (int t = 0; t < D && !any; ++t) any = dorow[t] != 0.0f;
            if (!any) continue;
            const double m = score_row(s, i, qrow, kb, n, D, (double)s->scale, p);
            double l = 0.0;
            for (int j = 0; j < n; ++j) { p[j] = exp(p[j] - m); l += p[j]; }
            double dl = 0.0;
            for (int j = 0; j < n; ++j) {
                p[j] /= l;
                const float* vr = vb + (size_t)j * D;
                double a = 0.0;
                for (int t = 0; t < D; ++t) a += (double)vr[t] * (double)dorow[t];
                dl += a * p[j];
            }
            for (int c = 0; c < n_cols; ++c) {
                const int j = cols[c];
                if (j >= n) continue;
                const float* vr = vb + (size_t)j * D;
                double a = 0.0;
                for (int t = 0; t < D; ++t) a += (double)vr[t] * (double)dorow[t];
                const double ds = p[j] * (a - dl) * (double)s->scale;
                for (int t = 0; t < D; ++t) {
                    dk_acc[(size_t)c * D + t] += ds * (double)qrow[t];
                    dv_acc[(size_t)c * D + t] += p[j] * (double)dorow[t];
                }
            }
        }
        free(p);
    }
    for (size_t e = 0; e < slab; ++e) {
        double a = 0.0, c = 0.0;
        for (int t = 0; t < threads; ++t) {
            a += dk_part[(size_t)t * slab * 2 + e];
            c += dk_part[(size_t)t * slab * 2 + slab + e];
        }
        dk_rows[e] = (float)a;
        dv_rows[e] = (float)c;
    }
    free(dk_part);
    return 0;
}

/* round-to-nearest-even fp32 -> bf16 -> fp32, the rounding the bf16 configs apply to their inputs */
void oracle_round_bf16(float* x, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, &x[i], 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) { u |= 0x00400000u; u &= 0xffff0000u; }
        else { u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u; }
        memcpy(&x[i], &u, 4);
    }
}

int oracle_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Rotary position embedding, restated from sentinel/NeuralNet/Layers/RotaryEmbedding.cpp: the angle tables (:19-27,
 * fp32 pow / cos / sin) and the in-place rotation of a feature-major (heads*head_dim) x cols matrix (:38-59; inverse
 * :61-81).  Column c sits at position (segment > 0 ? c % segment : position_offset + c), the rule of the reference's
 * device kernel (sentinel/NeuralNet/Cuda/CudaOps.cu:366).  fp32 arithmetic with separately rounded products and sums,
 * as the reference's host code computes: integer-exact parity is expected of anything compared with it.
 */
void oracle_rope_tables(int head_dim, int positions, float base, float* cos_t, float* sin_t)
{
    const int pairs = head_dim / 2;
    for (int pos = 0; pos < positions; ++pos)
        for (int i = 0; i < pairs; ++i) {
            const float exponent = -2.0f * (float)i / (float)head_dim;
            const float angle = (float)pos * powf(base, exponent);
            cos_t[(size_t)pos * pairs + i] = cosf(angle);
            sin_t[(size_t)pos * pairs + i] = sinf(angle);
        }
}

void oracle_rope_rotate(float* tensor, int heads, int head_dim, int cols, const float* cos_t, const float* sin_t,
                        int position_offset, int segment, int inverse)
{
    const int pairs = head_dim / 2;
    for (int h = 0; h < heads; ++h)
        for (int c = 0; c < cols; ++c) {
            const int pos = segment > 0 ? c % segment : position_offset + c;
            for (int i = 0; i < pairs; ++i) {
                float* even = tensor + ((size_t)h * head_dim + 2 * i) * cols + c;
                float* odd = even + cols;
                const float cs = cos_t[(size_t)pos * pairs + i], sn = sin_t[(size_t)pos * pairs + i];
                const float e = *even, o = *odd;
                if (!inverse) {
                    *even = e * cs - o * sn;
                    *odd = e * sn + o * cs;
                } else {
                    *even = e * cs + o * sn;
                    *odd = -e * sn + o * cs;
                }
            }
        }
}
