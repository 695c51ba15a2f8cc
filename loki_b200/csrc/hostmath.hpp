// Host-side vector math used to PREPARE QUERIES (O(dim) work per query; the corpus
// never passes through here).  Each function keeps the reference's operation order
// so that a prepared query is bit-identical to what the Go code would produce.
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <vector>

namespace lk {
namespace hm {

// media-server/embedvec/embedvec.go:34-50
inline void normalize(const float *x, int d, float *out) {
    double sum = 0.0;
    for (int i = 0; i < d; ++i) sum += (double)x[i] * (double)x[i];
    if (sum == 0.0) {
        if (out != x) memcpy(out, x, sizeof(float) * (size_t)d);
        return;
    }
    const double norm = sqrt(sum);
    for (int i = 0; i < d; ++i) out[i] = (float)((double)x[i] / norm);
}

// media-server/embedvec/embedvec.go:113-122
inline float cosine(const float *a, const float *b, int d) {
    double dot = 0.0;
    for (int i = 0; i < d; ++i) dot += (double)a[i] * (double)b[i];
    return (float)dot;
}

// Query side of centered scoring: qc = normalize(q_hat - mu), cq = <qc, mu>.
// media-server/embedindex/embedindex.go:291-296
inline float center_query(const float *q_hat, const float *mu, int d, float *qc) {
    std::vector<float> t((size_t)d);
    for (int i = 0; i < d; ++i) t[i] = q_hat[i] - mu[i];
    normalize(t.data(), d, qc);
    return cosine(qc, mu, d);
}

// Mean from the float64 column sum.  media-server/embedindex/embedindex.go:252-259
inline double mean_from_sum(const double *sum, int d, int64_t n, float *mu) {
    double n2 = 0.0;
    for (int i = 0; i < d; ++i) {
        const double m = sum[i] / (double)n;
        mu[i] = (float)m;
        n2 += m * m;
    }
    return n2;
}

// int8 quantisation of a normalised vector (this project's definition; the
// reference has no int8 path): scale = max|x|/127, code = clamp(rne(x/scale), -127, 127).
inline float quantize_i8(const float *x, int d, int8_t *q) {
    float amax = 0.0f;
    for (int i = 0; i < d; ++i) {
        const float a = fabsf(x[i]);
        if (a > amax) amax = a;
    }
    if (amax == 0.0f) {
        memset(q, 0, (size_t)d);
        return 0.0f;
    }
    const float s = amax / 127.0f;
    for (int i = 0; i < d; ++i) {
        float r = rintf(x[i] / s);
        if (r > 127.0f) r = 127.0f;
        if (r < -127.0f) r = -127.0f;
        q[i] = (int8_t)r;
    }
    return s;
}

}  // namespace hm
}  // namespace lk

namespace lk {
namespace hm {

// Host half of a shared-concept ("must match all") query: everything
// embedvec.NewSharedQuery computes (media-server/embedvec/shared.go:61-167), after the
// index-level normalise/centre step (media-server/embedindex/embedindex.go:343-357).
struct SharedPrep {
    int dim = 0, m = 0, rank = 0, nneg = 0;
    float gamma = 0.0f, lambda = 0.0f;
    std::vector<float> vecs;     // (m + rank + nneg) x dim: positives, basis, negatives
    std::vector<float> posw, posnorm, negw, qb;  // qb is m x rank
    int terms() const { return m + rank + nneg; }
};

// Returns 0, or 1 (no positives), 2 (a positive weight <= 0).
inline int shared_prepare(const float *pos, const float *posw, int npos, const float *neg, const float *negw,
                          int nneg, int d, float beta, float lambda, const float *mu, SharedPrep *out) {
    if (npos <= 0) return 1;
    if (beta < 0) beta = 0;
    if (beta > 1) beta = 1;
    if (lambda < 0) lambda = 0;
    SharedPrep &s = *out;
    s.dim = d;
    s.m = npos;
    s.nneg = nneg;
    s.rank = 0;
    s.gamma = beta * (2 - beta);
    s.lambda = lambda;
    std::vector<float> P((size_t)npos * d), N((size_t)std::max(nneg, 1) * d), t((size_t)d);
    auto prep = [&](const float *v, float *o) {
        normalize(v, d, o);
        if (mu) {
            for (int i = 0; i < d; ++i) t[i] = o[i] - mu[i];
            normalize(t.data(), d, o);
        }
        normalize(o, d, o);  // NewSharedQuery normalises its inputs once more
    };
    s.posw.assign((size_t)npos, 0.0f);
    s.posnorm.assign((size_t)npos, 0.0f);
    s.negw.assign((size_t)nneg, 0.0f);
    double wsum = 0.0;
    for (int i = 0; i < npos; ++i) {
        prep(pos + (size_t)i * d, &P[(size_t)i * d]);
        const float w = posw ? posw[i] : 1.0f;
        if (!(w > 0)) return 2;
        s.posw[i] = w;
        wsum += (double)w;
    }
    for (int i = 0; i < npos; ++i) s.posw[i] = (float)((double)s.posw[i] / wsum);
    for (int i = 0; i < nneg; ++i) {
        prep(neg + (size_t)i * d, &N[(size_t)i * d]);
        const float w = negw[i];
        s.negw[i] = w < 0 ? -w : w;
    }
    std::vector<float> B;
    if (beta > 0 && npos > 1) {
        std::vector<float> mean((size_t)d, 0.0f), diff((size_t)d);
        for (int i = 0; i < npos; ++i)
            for (int k = 0; k < d; ++k) mean[k] += P[(size_t)i * d + k] / (float)npos;
        for (int i = 0; i < npos; ++i) {
            for (int k = 0; k < d; ++k) diff[k] = P[(size_t)i * d + k] - mean[k];
            for (int j = 0; j < s.rank; ++j) {
                const float *b = &B[(size_t)j * d];
                const float proj = cosine(b, diff.data(), d);
                for (int k = 0; k < d; ++k) diff[k] -= proj * b[k];
            }
            double n2 = 0.0;
            for (int k = 0; k < d; ++k) n2 += (double)diff[k] * (double)diff[k];
            if (n2 < 1e-8) continue;
            B.resize((size_t)(s.rank + 1) * d);
            normalize(diff.data(), d, &B[(size_t)s.rank * d]);
            s.rank++;
        }
    }
    s.qb.assign((size_t)npos * std::max(s.rank, 1), 0.0f);
    for (int i = 0; i < npos; ++i) {
        double b2 = 0.0;
        for (int j = 0; j < s.rank; ++j) {
            const float dd = cosine(&P[(size_t)i * d], &B[(size_t)j * d], d);
            s.qb[(size_t)i * s.rank + j] = dd;
            b2 += (double)dd * (double)dd;
        }
        double n2 = 1.0 - (double)s.gamma * b2;
        if (n2 < 1e-6) n2 = 1e-6;
        s.posnorm[i] = (float)sqrt(n2);
    }
    s.vecs.clear();
    s.vecs.insert(s.vecs.end(), P.begin(), P.end());
    s.vecs.insert(s.vecs.end(), B.begin(), B.end());
    if (nneg > 0) s.vecs.insert(s.vecs.end(), N.begin(), N.begin() + (size_t)nneg * d);
    return 0;
}

}  // namespace hm
}  // namespace lk
