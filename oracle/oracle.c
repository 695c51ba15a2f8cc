/*
 * CPU oracle for the exact vector-scan path.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped library links, loads or calls this file.  It restates, in plain
 * C, the arithmetic of the reference's Go packages so that the CUDA kernels can
 * be checked against it on identical inputs.
 *
 * Parity status
 *   fp32 path (normalize, cosine, centered cosine, heap top-k, shared query):
 *     pinned against the literal-vector known-answer tests of the reference
 *     (the _test.go files of media-server/embedindex and media-server/embedvec); the
 *     Go toolchain is not available, so the reference itself is never executed.
 *   int8 quantise / int32 scan and 64-bit Hamming: PARITY UNPINNED.  The
 *     reference has no such code; these functions restate the definitions this
 *     project fixes (see each function) and are cross-checked by an independent
 *     numpy implementation in the tests.
 *
 * Build: see oracle/Makefile (gcc -O2, no -ffast-math, -ffp-contract=off).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* embedvec                                                                  */
/* ------------------------------------------------------------------------- */

/* L2-normalise: f64 sum of squares in index order, out[i] = (float)((double)x[i]/norm);
 * a zero vector is copied unchanged.  Follows media-server/embedvec/embedvec.go:34-50. */
ORC_API void orc_normalize(const float *x, int d, float *out) {
    double sum = 0.0;
    for (int i = 0; i < d; i++) sum += (double)x[i] * (double)x[i];
    if (sum == 0.0) {
        memcpy(out, x, (size_t)d * sizeof(float));
        return;
    }
    double norm = sqrt(sum);
    for (int i = 0; i < d; i++) out[i] = (float)((double)x[i] / norm);
}

/* Dot product, f32 in, f64 accumulate in index order, one rounding to f32.
 * Follows media-server/embedvec/embedvec.go:113-122 (length check is the caller's). */
ORC_API float orc_cosine(const float *a, const float *b, int d) {
    double dot = 0.0;
    for (int i = 0; i < d; i++) dot += (double)a[i] * (double)b[i];
    return (float)dot;
}

/* True cosine of un-normalised inputs; 0 when either is a zero vector.
 * Follows media-server/embedvec/embedvec.go:127-141. */
ORC_API float orc_cosine_sim(const float *a, const float *b, int d) {
    double dot = 0.0, na = 0.0, nb = 0.0;
    for (int i = 0; i < d; i++) {
        dot += (double)a[i] * (double)b[i];
        na += (double)a[i] * (double)a[i];
        nb += (double)b[i] * (double)b[i];
    }
    if (na == 0.0 || nb == 0.0) return 0.0f;
    return (float)(dot / (sqrt(na) * sqrt(nb)));
}

/* ------------------------------------------------------------------------- */
/* embedindex: scorers                                                       */
/* ------------------------------------------------------------------------- */

/* ||v - mu|| for unit v: sqrt(max(0, 1 - 2*<v,mu> + muN2)) with <v,mu> first rounded
 * to f32.  Follows media-server/embedindex/embedindex.go:222-228. */
ORC_API float orc_centered_norm(const float *v, const float *mu, int d, double mu_n2) {
    double n2 = 1.0 - 2.0 * (double)orc_cosine(v, mu, d) + mu_n2;
    if (n2 < 0.0) n2 = 0.0;
    return (float)sqrt(n2);
}

/* Mean vector from the f64 running column sum: m = sum/n, mu = (float)m, muN2 = sum m*m.
 * Follows media-server/embedindex/embedindex.go:252-259. */
ORC_API double orc_mean_from_sum(const double *sum, int d, int64_t n, float *mu) {
    double n2 = 0.0;
    for (int i = 0; i < d; i++) {
        double m = sum[i] / (double)n;
        mu[i] = (float)m;
        n2 += m * m;
    }
    return n2;
}

/* Query preparation for centered scoring: qc = normalize(q_hat - mu) (f32 subtract),
 * cq = cosine(qc, mu).  Follows media-server/embedindex/embedindex.go:291-296. */
ORC_API float orc_center_query(const float *q_hat, const float *mu, int d, float *qc) {
    float *t = (float *)malloc((size_t)d * sizeof(float));
    for (int i = 0; i < d; i++) t[i] = q_hat[i] - mu[i];
    orc_normalize(t, d, qc);
    free(t);
    return orc_cosine(qc, mu, d);
}

/* One centered score, f32 epilogue: cn < 1e-6 -> 0, else (cosine(qc,v) - cq) / cn.
 * Follows media-server/embedindex/embedindex.go:297-305. */
static inline float centered_score(const float *qc, const float *v, int d, float cq, float cn) {
    if (cn < 1e-6f) return 0.0f;
    float dot = orc_cosine(qc, v, d);
    float diff = dot - cq;
    return diff / cn;
}

typedef struct {
    const float *rows;      /* contiguous arena (ld floats per row), or NULL */
    const float *const *rowp; /* one pointer per row (the reference's layout), or NULL */
    int64_t ld;
    int d;
    const float *q;
    const float *cnorm;     /* NULL = plain scoring */
    float cq;
    const int32_t *slots;   /* NULL = every row */
    float *scores;
    int64_t lo, hi;
} scan_job;

static void *scan_worker(void *arg) {
    scan_job *j = (scan_job *)arg;
    for (int64_t t = j->lo; t < j->hi; t++) {
        int64_t s = j->slots ? (int64_t)j->slots[t] : t;
        const float *v = j->rowp ? j->rowp[s] : j->rows + s * j->ld;
        j->scores[t] = j->cnorm ? centered_score(j->q, v, j->d, j->cq, j->cnorm[s])
                                : orc_cosine(j->q, v, j->d);
    }
    return NULL;
}

/* Score n candidates (all rows, or rows[slots[t]]) into scores[t], split into
 * `workers` contiguous chunks, one thread each, chunk = ceil(n/workers).
 * Follows media-server/embedindex/embedindex.go:432-442 and :460-479. */
ORC_API void orc_scan_f32(const float *rows, const float *const *rowp, int64_t ld, int d,
                          const float *q, const float *cnorm, float cq,
                          const int32_t *slots, int64_t n, float *scores, int workers) {
    if (n <= 0) return;
    if (workers < 1) workers = 1;
    if ((int64_t)workers > n) workers = (int)n;
    int64_t chunk = (n + workers - 1) / workers;
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)workers);
    scan_job *jobs = (scan_job *)malloc(sizeof(scan_job) * (size_t)workers);
    int nj = 0;
    for (int64_t lo = 0; lo < n; lo += chunk, nj++) {
        int64_t hi = lo + chunk > n ? n : lo + chunk;
        scan_job jb = {rows, rowp, ld, d, q, cnorm, cq, slots, scores, lo, hi};
        jobs[nj] = jb;
        if (workers == 1) scan_worker(&jobs[nj]);
        else pthread_create(&th[nj], NULL, scan_worker, &jobs[nj]);
    }
    if (workers > 1)
        for (int i = 0; i < nj; i++) pthread_join(th[i], NULL);
    free(th);
    free(jobs);
}

/* ------------------------------------------------------------------------- */
/* embedindex: top-k                                                         */
/* ------------------------------------------------------------------------- */

/* Size-k min-heap of indices over scores; a later score replaces the root only
 * when strictly greater.  Returns the heap array (heap order, not sorted).
 * Follows media-server/embedindex/embedindex.go:495-534. */
ORC_API int orc_topk_heap_f32(const float *scores, int64_t n, int k, int32_t *h) {
    int len = 0;
    for (int64_t i = 0; i < n; i++) {
        if (len < k) {
            int pos = len;
            h[len++] = (int32_t)i;
            while (pos > 0) { /* sift up */
                int parent = (pos - 1) / 2;
                if (scores[h[parent]] <= scores[h[pos]]) break;
                int32_t t = h[pos]; h[pos] = h[parent]; h[parent] = t;
                pos = parent;
            }
        } else if (k > 0 && scores[i] > scores[h[0]]) {
            h[0] = (int32_t)i;
            int pos = 0;
            for (;;) { /* sift down */
                int l = 2 * pos + 1, r = 2 * pos + 2, small = pos;
                if (l < len && scores[h[l]] < scores[h[small]]) small = l;
                if (r < len && scores[h[r]] < scores[h[small]]) small = r;
                if (small == pos) break;
                int32_t t = h[pos]; h[pos] = h[small]; h[small] = t;
                pos = small;
            }
        }
    }
    return len;
}

/* ------------------------------------------------------------------------- */
/* embedvec.SharedQuery                                                      */
/* ------------------------------------------------------------------------- */

#define ORC_SHARED_MAX 64

typedef struct {
    int d, m, rank, nneg;
    float gamma, lambda;
    float *pos;    /* m x d, unit */
    float *neg;    /* nneg x d, unit */
    float *basis;  /* rank x d, orthonormal */
    float posw[ORC_SHARED_MAX];
    float negw[ORC_SHARED_MAX];
    float posnorm[ORC_SHARED_MAX];
    float *qb;     /* m x rank */
} orc_shared;

ORC_API void orc_shared_free(orc_shared *s) {
    if (!s) return;
    free(s->pos); free(s->neg); free(s->basis); free(s->qb); free(s);
}

/* Build the shared-concept scorer.  Returns NULL and sets *err (1 no positives,
 * 2 non-positive weight, 3 too many terms) on invalid input; weight-count and
 * dimension mismatches are rejected by the caller, which owns the ragged inputs.
 * posw == NULL means equal weights.  Follows media-server/embedvec/shared.go:61-167. */
ORC_API orc_shared *orc_shared_new(const float *pos, const float *posw, int m,
                                   const float *neg, const float *negw, int nneg,
                                   int d, float beta, float lambda, int *err) {
    *err = 0;
    if (m <= 0) { *err = 1; return NULL; }
    if (m > ORC_SHARED_MAX || nneg > ORC_SHARED_MAX) { *err = 3; return NULL; }
    if (beta < 0) beta = 0;
    if (beta > 1) beta = 1;
    if (lambda < 0) lambda = 0;
    orc_shared *s = (orc_shared *)calloc(1, sizeof(orc_shared));
    s->d = d; s->m = m; s->nneg = nneg;
    s->gamma = beta * (2 - beta);
    s->lambda = lambda;
    s->pos = (float *)malloc(sizeof(float) * (size_t)m * d);
    s->neg = (float *)malloc(sizeof(float) * (size_t)(nneg > 0 ? nneg : 1) * d);
    s->basis = (float *)malloc(sizeof(float) * (size_t)m * d);
    double wsum = 0.0;
    for (int i = 0; i < m; i++) {
        orc_normalize(pos + (size_t)i * d, d, s->pos + (size_t)i * d);
        float w = posw ? posw[i] : 1.0f;
        if (!(w > 0)) { *err = 2; orc_shared_free(s); return NULL; }
        s->posw[i] = w;
        wsum += (double)w;
    }
    for (int i = 0; i < m; i++) s->posw[i] = (float)((double)s->posw[i] / wsum);
    for (int i = 0; i < nneg; i++) {
        orc_normalize(neg + (size_t)i * d, d, s->neg + (size_t)i * d);
        float w = negw[i];
        s->negw[i] = w < 0 ? -w : w;
    }
    /* variation subspace: modified Gram-Schmidt over offsets from the f32 mean */
    if (beta > 0 && m > 1) {
        float *mean = (float *)calloc((size_t)d, sizeof(float));
        float *diff = (float *)malloc(sizeof(float) * (size_t)d);
        for (int i = 0; i < m; i++)
            for (int k = 0; k < d; k++) mean[k] += s->pos[(size_t)i * d + k] / (float)m;
        for (int i = 0; i < m; i++) {
            for (int k = 0; k < d; k++) diff[k] = s->pos[(size_t)i * d + k] - mean[k];
            for (int j = 0; j < s->rank; j++) {
                const float *b = s->basis + (size_t)j * d;
                float proj = orc_cosine(b, diff, d);
                for (int k = 0; k < d; k++) diff[k] -= proj * b[k];
            }
            double n2 = 0.0;
            for (int k = 0; k < d; k++) n2 += (double)diff[k] * (double)diff[k];
            if (n2 < 1e-8) continue;
            orc_normalize(diff, d, s->basis + (size_t)s->rank * d);
            s->rank++;
        }
        free(mean); free(diff);
    }
    s->qb = (float *)malloc(sizeof(float) * (size_t)m * (size_t)(s->rank > 0 ? s->rank : 1));
    for (int i = 0; i < m; i++) {
        double b2 = 0.0;
        for (int j = 0; j < s->rank; j++) {
            float dd = orc_cosine(s->pos + (size_t)i * d, s->basis + (size_t)j * d, d);
            s->qb[(size_t)i * s->rank + j] = dd;
            b2 += (double)dd * (double)dd;
        }
        double n2 = 1.0 - (double)s->gamma * b2;
        if (n2 < 1e-6) n2 = 1e-6;
        s->posnorm[i] = (float)sqrt(n2);
    }
    return s;
}

ORC_API int orc_shared_rank(const orc_shared *s) { return s->rank; }
/* Copies the prepared terms out (used to cross-check the library's host-side prep). */
ORC_API void orc_shared_export(const orc_shared *s, float *pos, float *basis, float *posw,
                               float *posnorm, float *qb, float *gamma) {
    memcpy(pos, s->pos, sizeof(float) * (size_t)s->m * s->d);
    memcpy(basis, s->basis, sizeof(float) * (size_t)s->rank * s->d);
    memcpy(posw, s->posw, sizeof(float) * (size_t)s->m);
    memcpy(posnorm, s->posnorm, sizeof(float) * (size_t)s->m);
    memcpy(qb, s->qb, sizeof(float) * (size_t)s->m * s->rank);
    *gamma = s->gamma;
}

/* Score one unit candidate.  Follows media-server/embedvec/shared.go:180-220. */
ORC_API float orc_shared_score(const orc_shared *s, const float *v) {
    float vb[ORC_SHARED_MAX];
    double sc[ORC_SHARED_MAX];
    int d = s->d;
    double b2 = 0.0;
    for (int j = 0; j < s->rank; j++) {
        float dd = orc_cosine(s->basis + (size_t)j * d, v, d);
        vb[j] = dd;
        b2 += (double)dd * (double)dd;
    }
    double vn2 = 1.0 - (double)s->gamma * b2;
    if (vn2 < 1e-6) vn2 = 1e-6;
    double vn = sqrt(vn2);
    double mean = 0.0, m2 = 0.0;
    for (int i = 0; i < s->m; i++) {
        double x = (double)orc_cosine(s->pos + (size_t)i * d, v, d);
        for (int j = 0; j < s->rank; j++)
            x -= (double)s->gamma * (double)s->qb[(size_t)i * s->rank + j] * (double)vb[j];
        x /= (double)s->posnorm[i] * vn;
        sc[i] = x;
        mean += (double)s->posw[i] * x;
    }
    for (int i = 0; i < s->m; i++) {
        double dd = sc[i] - mean;
        m2 += (double)s->posw[i] * dd * dd;
    }
    double out = mean - (double)s->lambda * sqrt(m2);
    for (int i = 0; i < s->nneg; i++)
        out -= (double)s->negw[i] * (double)orc_cosine(s->neg + (size_t)i * d, v, d);
    return (float)out;
}

/* Shared-concept scan over n candidates; with mu != NULL each candidate is first
 * re-expressed as (v - mu) * (1/cnorm) in f32, cnorm < 1e-6 scoring 0.
 * Follows media-server/embedindex/embedindex.go:374-393. */
ORC_API void orc_scan_shared(const orc_shared *s, const float *rows, int64_t ld,
                             const float *mu, const float *cnorm,
                             const int32_t *slots, int64_t n, float *scores) {
    int d = s->d;
    float *scratch = (float *)malloc(sizeof(float) * (size_t)(d > 0 ? d : 1));
    for (int64_t t = 0; t < n; t++) {
        int64_t sl = slots ? (int64_t)slots[t] : t;
        const float *v = rows + sl * ld;
        if (!mu) { scores[t] = orc_shared_score(s, v); continue; }
        float cn = cnorm[sl];
        if (cn < 1e-6f) { scores[t] = 0.0f; continue; }
        float inv = 1.0f / cn;
        for (int k = 0; k < d; k++) scratch[k] = (v[k] - mu[k]) * inv;
        scores[t] = orc_shared_score(s, scratch);
    }
    free(scratch);
}

/* ------------------------------------------------------------------------- */
/* int8 path (no counterpart in the reference; definitions fixed by this project) */
/* ------------------------------------------------------------------------- */

/* Quantise an already L2-normalised row: scale = max|x| / 127 (f32 divide);
 * code = clamp(round-half-even(x / scale), -127, 127) (f32 divide); a zero row
 * gives scale 0 and all-zero codes. */
ORC_API void orc_quantize_i8(const float *x, int d, int8_t *q, float *scale) {
    float amax = 0.0f;
    for (int i = 0; i < d; i++) {
        float a = fabsf(x[i]);
        if (a > amax) amax = a;
    }
    if (amax == 0.0f) {
        memset(q, 0, (size_t)d);
        *scale = 0.0f;
        return;
    }
    float s = amax / 127.0f;
    for (int i = 0; i < d; i++) {
        float r = rintf(x[i] / s); /* default rounding mode: to nearest, ties to even */
        if (r > 127.0f) r = 127.0f;
        if (r < -127.0f) r = -127.0f;
        q[i] = (int8_t)r;
    }
    *scale = s;
}

/* Normalise then quantise n rows (ld_in floats apart) into codes (ld_out bytes apart,
 * padding bytes zeroed). */
ORC_API void orc_build_i8(const float *rows, int64_t n, int d, int64_t ld_in,
                          int8_t *codes, int64_t ld_out, float *scales) {
    float *t = (float *)malloc(sizeof(float) * (size_t)(d > 0 ? d : 1));
    for (int64_t i = 0; i < n; i++) {
        orc_normalize(rows + i * ld_in, d, t);
        int8_t *c = codes + i * ld_out;
        orc_quantize_i8(t, d, c, &scales[i]);
        for (int64_t k = d; k < ld_out; k++) c[k] = 0;
    }
    free(t);
}

/* int32-accumulated dot of int8 codes for every row (or rows[slots[t]]). */
ORC_API void orc_scan_i8(const int8_t *codes, int64_t ld, int d, const int8_t *q,
                         const int32_t *slots, int64_t n, int32_t *scores) {
    for (int64_t t = 0; t < n; t++) {
        const int8_t *v = codes + (slots ? (int64_t)slots[t] : t) * ld;
        int32_t acc = 0;
        for (int k = 0; k < d; k++) acc += (int32_t)v[k] * (int32_t)q[k];
        scores[t] = acc;
    }
}

/* Exact top-k by (score descending, id ascending); ids[t] names candidate t
 * (NULL = t itself).  Writes k' = min(k, n) entries in rank order. */
typedef struct { int64_t key; int32_t id; } kv_t;
static int kv_cmp(const void *a, const void *b) {
    const kv_t *x = (const kv_t *)a, *y = (const kv_t *)b;
    if (x->key != y->key) return x->key > y->key ? -1 : 1;
    if (x->id != y->id) return x->id < y->id ? -1 : 1;
    return 0;
}
ORC_API int orc_topk_i32(const int32_t *scores, const int32_t *ids, int64_t n, int k,
                         int32_t *out_ids, int32_t *out_scores) {
    if (n <= 0 || k <= 0) return 0;
    kv_t *a = (kv_t *)malloc(sizeof(kv_t) * (size_t)n);
    for (int64_t i = 0; i < n; i++) { a[i].key = scores[i]; a[i].id = ids ? ids[i] : (int32_t)i; }
    qsort(a, (size_t)n, sizeof(kv_t), kv_cmp);
    int kk = k < n ? k : (int)n;
    for (int i = 0; i < kk; i++) { out_ids[i] = a[i].id; out_scores[i] = (int32_t)a[i].key; }
    free(a);
    return kk;
}

/* Same ordering rule for f32 scores (-0 ranks equal to +0; NaN is not supported). */
typedef struct { float key; int32_t id; } kvf_t;
static int kvf_cmp(const void *a, const void *b) {
    const kvf_t *x = (const kvf_t *)a, *y = (const kvf_t *)b;
    if (x->key != y->key) return x->key > y->key ? -1 : 1;
    if (x->id != y->id) return x->id < y->id ? -1 : 1;
    return 0;
}
ORC_API int orc_topk_f32(const float *scores, const int32_t *ids, int64_t n, int k,
                         int32_t *out_ids, float *out_scores) {
    if (n <= 0 || k <= 0) return 0;
    kvf_t *a = (kvf_t *)malloc(sizeof(kvf_t) * (size_t)n);
    for (int64_t i = 0; i < n; i++) { a[i].key = scores[i]; a[i].id = ids ? ids[i] : (int32_t)i; }
    qsort(a, (size_t)n, sizeof(kvf_t), kvf_cmp);
    int kk = k < n ? k : (int)n;
    for (int i = 0; i < kk; i++) { out_ids[i] = a[i].id; out_scores[i] = a[i].key; }
    free(a);
    return kk;
}

/* ------------------------------------------------------------------------- */
/* 64-bit Hamming (no counterpart in the reference)                          */
/* ------------------------------------------------------------------------- */

/* All pairs i<j with popcount(h[i]^h[j]) <= radius whose i lies in [i_lo, i_hi), in
 * lexicographic (i,j) order.  Writes at most cap pairs; returns the number found.  Row ranges
 * are independent, so a caller may run several on threads and concatenate them in order. */
ORC_API int64_t orc_hamming_pairs_rows(const uint64_t *h, int64_t n, int radius, int64_t i_lo, int64_t i_hi,
                                       uint32_t *pairs, int64_t cap) {
    int64_t cnt = 0;
    for (int64_t i = i_lo; i < i_hi && i < n; i++) {
        uint64_t a = h[i];
        for (int64_t j = i + 1; j < n; j++) {
            if (__builtin_popcountll(a ^ h[j]) <= radius) {
                if (cnt < cap) { pairs[2 * cnt] = (uint32_t)i; pairs[2 * cnt + 1] = (uint32_t)j; }
                cnt++;
            }
        }
    }
    return cnt;
}

/* All pairs i<j with popcount(h[i]^h[j]) <= radius, in lexicographic (i,j) order.
 * Writes at most cap pairs; returns the total found. */
ORC_API int64_t orc_hamming_pairs(const uint64_t *h, int64_t n, int radius,
                                  uint32_t *pairs, int64_t cap) {
    return orc_hamming_pairs_rows(h, n, radius, 0, n, pairs, cap);
}

/* One hash against n: distances out. */
ORC_API void orc_hamming_scan(const uint64_t *h, int64_t n, uint64_t q, int32_t *dist) {
    for (int64_t i = 0; i < n; i++) dist[i] = __builtin_popcountll(h[i] ^ q);
}

/* ------------------------------------------------------------------------- */
/* tasks/face_cluster.go: the all-pairs neighbour prescreen of face clustering  */
/* ------------------------------------------------------------------------- */

/* float32 dot with four interleaved accumulators, combined (s0+s1)+(s2+s3).
 * Follows media-server/tasks/face_cluster.go:908-925 (equal lengths assumed). */
ORC_API float orc_dotf(const float *a, const float *b, int n) {
    float s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    int i = 0;
    for (; i + 4 <= n; i += 4) {
        s0 += a[i] * b[i];
        s1 += a[i + 1] * b[i + 1];
        s2 += a[i + 2] * b[i + 2];
        s3 += a[i + 3] * b[i + 3];
    }
    for (; i < n; i++) s0 += a[i] * b[i];
    return (s0 + s1) + (s2 + s3);
}

/* b against four rows at once: even elements into s, odd into t, result s + t.
 * Follows media-server/tasks/face_cluster.go:939-967. */
static void dot4(const float *a0, const float *a1, const float *a2, const float *a3, const float *b, int n,
                 float out[4]) {
    float s0 = 0, s1 = 0, s2 = 0, s3 = 0, t0 = 0, t1 = 0, t2 = 0, t3 = 0;
    int i = 0;
    for (; i + 2 <= n; i += 2) {
        float x = b[i], y = b[i + 1];
        s0 += a0[i] * x; t0 += a0[i + 1] * y;
        s1 += a1[i] * x; t1 += a1[i + 1] * y;
        s2 += a2[i] * x; t2 += a2[i + 1] * y;
        s3 += a3[i] * x; t3 += a3[i + 1] * y;
    }
    for (; i < n; i++) {
        float x = b[i];
        s0 += a0[i] * x; s1 += a1[i] * x; s2 += a2[i] * x; s3 += a3[i] * x;
    }
    out[0] = s0 + t0; out[1] = s1 + t1; out[2] = s2 + t2; out[3] = s3 + t3;
}

#define ORC_MAX_FORM 256 /* maxFormCandidates, media-server/tasks/face_cluster.go:1156 */

/* For every row i the earlier rows j < i with dot >= threshold, ascending, at most 256;
 * a row with more is marked overflow and its list dropped.  near is n x 256 int32,
 * count n int32, overflow n bytes.  Row tiles of 64, column tiles ascending, four rows at a
 * time through dot4 off the diagonal, dotf elsewhere: follows
 * media-server/tasks/face_cluster.go:1189-1285 (the result does not depend on how the
 * reference's workers interleave: a row tile belongs to one worker). */
ORC_API void orc_prescreen(const float *v, int n, int d, float threshold, int32_t *near, int32_t *count,
                           uint8_t *overflow) {
    const int tile = 64;
    memset(count, 0, sizeof(int32_t) * (size_t)n);
    memset(overflow, 0, (size_t)n);
    /* lists may transiently hold more than 256 entries inside the four-row fast path */
    int32_t *tmp = (int32_t *)malloc(sizeof(int32_t) * (size_t)n * (ORC_MAX_FORM + tile + 1));
    const size_t ts = ORC_MAX_FORM + tile + 1;
    for (int iLo = 0; iLo < n; iLo += tile) {
        int iHi = iLo + tile < n ? iLo + tile : n;
        for (int jLo = 0; jLo < iHi; jLo += tile) {
            int jHi = jLo + tile < iHi ? jLo + tile : iHi;
            int i = iLo;
            if (jHi <= iLo) {
                for (; i + 4 <= iHi; i += 4) {
                    if (overflow[i] || overflow[i + 1] || overflow[i + 2] || overflow[i + 3]) break;
                    for (int j = jLo; j < jHi; j++) {
                        float s[4];
                        dot4(v + (size_t)i * d, v + (size_t)(i + 1) * d, v + (size_t)(i + 2) * d,
                             v + (size_t)(i + 3) * d, v + (size_t)j * d, d, s);
                        for (int r = 0; r < 4; r++)
                            if (s[r] >= threshold) tmp[(size_t)(i + r) * ts + count[i + r]++] = j;
                    }
                    for (int r = i; r < i + 4; r++)
                        if (count[r] > ORC_MAX_FORM) { overflow[r] = 1; count[r] = 0; }
                }
            }
            for (; i < iHi; i++) {
                if (overflow[i]) continue;
                int jEnd = jHi < i ? jHi : i;
                for (int j = jLo; j < jEnd; j++) {
                    if (orc_dotf(v + (size_t)i * d, v + (size_t)j * d, d) < threshold) continue;
                    if (count[i] == ORC_MAX_FORM) { overflow[i] = 1; count[i] = 0; break; }
                    tmp[(size_t)i * ts + count[i]++] = j;
                }
            }
        }
    }
    for (int i = 0; i < n; i++)
        memcpy(near + (size_t)i * ORC_MAX_FORM, tmp + (size_t)i * ts, sizeof(int32_t) * (size_t)count[i]);
    free(tmp);
}

/* Every candidate against every seed, float32, in the reference's two summation orders:
 * inside each worker chunk candidates go four at a time through dot4 and the last one to three
 * through dotf.  out is n_cand x n_seeds.  chunk = candidates per worker chunk (0 = one chunk).
 * Follows media-server/tasks/face_cluster.go:1349-1360 and :1375-1400. */
ORC_API void orc_seed_scores(const float *cands, int n_cand, const float *seeds, int n_seeds, int d, int chunk,
                             float *out) {
    if (chunk <= 0) chunk = n_cand;
    for (int lo = 0; lo < n_cand; lo += chunk) {
        int hi = lo + chunk < n_cand ? lo + chunk : n_cand;
        int base = lo;
        for (; base + 4 <= hi; base += 4) {
            for (int k = 0; k < n_seeds; k++) {
                float s[4];
                dot4(cands + (size_t)base * d, cands + (size_t)(base + 1) * d, cands + (size_t)(base + 2) * d,
                     cands + (size_t)(base + 3) * d, seeds + (size_t)k * d, d, s);
                for (int r = 0; r < 4; r++) out[(size_t)(base + r) * n_seeds + k] = s[r];
            }
        }
        for (; base < hi; base++)
            for (int k = 0; k < n_seeds; k++)
                out[(size_t)base * n_seeds + k] = orc_dotf(cands + (size_t)base * d, seeds + (size_t)k * d, d);
    }
}

/* The one-candidate-at-a-time scores the reference's own test compares the grouped version
 * with (media-server/tasks/face_score_kernel_test.go:17-44): dotf for every pair. */
ORC_API void orc_seed_scores_single(const float *cands, int n_cand, const float *seeds, int n_seeds, int d, float *out) {
    for (int i = 0; i < n_cand; i++)
        for (int k = 0; k < n_seeds; k++)
            out[(size_t)i * n_seeds + k] = orc_dotf(cands + (size_t)i * d, seeds + (size_t)k * d, d);
}

/* float64-accumulated dot rounded once (media-server/tasks/face_cluster.go:890-896). */
ORC_API float orc_dot32(const float *a, const float *b, int n) {
    double acc = 0.0;
    for (int i = 0; i < n; i++) acc += (double)a[i] * (double)b[i];
    return (float)acc;
}

/* The definition the reference's own test checks the prescreen against
 * (media-server/tasks/face_cluster_perf_test.go:52-81): every j < i with dotf >= threshold. */
ORC_API void orc_prescreen_bruteforce(const float *v, int n, int d, float threshold, int32_t *near,
                                      int32_t *count, uint8_t *overflow) {
    for (int i = 0; i < n; i++) {
        int c = 0;
        overflow[i] = 0;
        for (int j = 0; j < i; j++) {
            if (orc_dotf(v + (size_t)i * d, v + (size_t)j * d, d) >= threshold) {
                if (c < ORC_MAX_FORM) near[(size_t)i * ORC_MAX_FORM + c] = j;
                c++;
            }
        }
        if (c > ORC_MAX_FORM) { overflow[i] = 1; c = 0; }
        count[i] = c;
    }
}

/* ------------------------------------------------------------------------- */
/* embedvec/pca.go: three-component PCA projection                              */
/* ------------------------------------------------------------------------- */

static double pca_dot(const double *a, const double *b, int d) { /* pca.go:209-215 */
    double s = 0;
    for (int i = 0; i < d; i++) s += a[i] * b[i];
    return s;
}
static void pca_orthogonalize(double *v, double *const *basis, int nb, int d) { /* pca.go:198-206 */
    for (int b = 0; b < nb; b++) {
        double p = pca_dot(v, basis[b], d);
        for (int j = 0; j < d; j++) v[j] -= p * basis[b][j];
    }
}
static double pca_normalize(double *v, int d) { /* pca.go:218-226 */
    double n = sqrt(pca_dot(v, v, d));
    if (n == 0) return 0;
    for (int j = 0; j < d; j++) v[j] /= n;
    return n;
}
/* u = Xc^T (Xc v) with on-the-fly centering; rows split into `workers` contiguous chunks whose
 * partial sums are merged in chunk order (pca.go:130-182). */
static void pca_cov_times(const float *x, int n, int d, const double *mean, const double *v, int workers, double *u) {
    double mv = pca_dot(mean, v, d);
    if (workers > n) workers = n;
    int chunk = (n + workers - 1) / workers;
    int nparts = (n + chunk - 1) / chunk;
    double *pu = (double *)calloc((size_t)nparts * d, sizeof(double));
    double *py = (double *)calloc((size_t)nparts, sizeof(double));
    for (int w = 0, lo = 0; lo < n; w++, lo += chunk) {
        int hi = lo + chunk < n ? lo + chunk : n;
        double *uw = pu + (size_t)w * d;
        double ysum = 0;
        for (int i = lo; i < hi; i++) {
            const float *row = x + (size_t)i * d;
            double y = 0;
            for (int j = 0; j < d; j++) y += (double)row[j] * v[j];
            y -= mv;
            ysum += y;
            for (int j = 0; j < d; j++) uw[j] += y * (double)row[j];
        }
        py[w] = ysum;
    }
    double ysum = 0;
    for (int j = 0; j < d; j++) u[j] = 0;
    for (int w = 0; w < nparts; w++) {
        ysum += py[w];
        for (int j = 0; j < d; j++) u[j] += pu[(size_t)w * d + j];
    }
    for (int j = 0; j < d; j++) u[j] -= ysum * mean[j];
    free(pu);
    free(py);
}

/* ProjectPCA3 (pca.go:22-128).  coords is n x 3 float32, variance 3 doubles; `workers` stands
 * for runtime.NumCPU() of the machine the reference runs on. */
ORC_API void orc_pca3(const float *x, int n, int d, int workers, float *coords, double *variance) {
    for (int i = 0; i < n * 3; i++) coords[i] = 0;
    variance[0] = variance[1] = variance[2] = 0;
    if (n == 0 || d == 0) return;
    if (workers < 1) workers = 1;
    double *mean = (double *)calloc((size_t)d, sizeof(double));
    for (int i = 0; i < n; i++)
        for (int j = 0; j < d; j++) mean[j] += (double)x[(size_t)i * d + j];
    for (int j = 0; j < d; j++) mean[j] /= (double)n;
    double total = 0;
    for (int i = 0; i < n; i++)
        for (int j = 0; j < d; j++) {
            double dx = (double)x[(size_t)i * d + j] - mean[j];
            total += dx * dx;
        }
    total /= (double)n;
    if (total == 0) { free(mean); return; }
    double *comps[3] = {0, 0, 0};
    double eigen[3] = {0, 0, 0};
    int nc = 0;
    double *u = (double *)malloc(sizeof(double) * (size_t)d);
    for (int c = 0; c < 3; c++) {
        double *v = (double *)malloc(sizeof(double) * (size_t)d);
        uint64_t state = 0x9E3779B97F4A7C15ull + (uint64_t)c * 0xBF58476D1CE4E5B9ull; /* pca.go:187-195 */
        for (int j = 0; j < d; j++) {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            v[j] = (double)(int64_t)(state >> 11) / (double)(1ull << 52) - 1;
        }
        pca_orthogonalize(v, comps, nc, d);
        if (pca_normalize(v, d) == 0) { free(v); break; }
        double lambda = 0;
        for (int iter = 0; iter < 100; iter++) {
            pca_cov_times(x, n, d, mean, v, workers, u);
            pca_orthogonalize(u, comps, nc, d);
            lambda = pca_normalize(u, d);
            if (lambda == 0) break;
            int done = fabs(pca_dot(u, v, d)) > 1 - 1e-10;
            memcpy(v, u, sizeof(double) * (size_t)d);
            if (done) break;
        }
        if (lambda == 0) { free(v); break; }
        comps[nc] = v;
        eigen[nc] = lambda / (double)n;
        nc++;
    }
    double mean_dot[3] = {0, 0, 0};
    for (int c = 0; c < nc; c++) mean_dot[c] = pca_dot(mean, comps[c], d);
    double max_abs = 0;
    for (int i = 0; i < n; i++)
        for (int c = 0; c < nc; c++) {
            double sacc = 0;
            for (int j = 0; j < d; j++) sacc += (double)x[(size_t)i * d + j] * comps[c][j];
            sacc -= mean_dot[c];
            coords[(size_t)i * 3 + c] = (float)sacc;
            if (fabs(sacc) > max_abs) max_abs = fabs(sacc);
        }
    if (max_abs > 0) {
        float sc = (float)(1 / max_abs);
        for (int i = 0; i < n * 3; i++) coords[i] *= sc;
    }
    for (int c = 0; c < nc; c++) variance[c] = eigen[c] / total;
    for (int c = 0; c < nc; c++) free(comps[c]);
    free(u);
    free(mean);
}
