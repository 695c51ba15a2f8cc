// Path-keyed index (include/lokiscan_index.h): the reference's exactIndex bookkeeping
// (media-server/embedindex/embedindex.go:122-140, :176-219, :398-419, :483-490) in C++,
// on top of the slot-level C ABI.  Vectors live in HBM only; this layer owns the
// path table, the slot map and the ordering of ties by path.
#include <algorithm>
#include <new>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/lokiscan_index.h"
#include "lk_common.cuh"

namespace lk {  // index.cu
int cache_identity(const char *path, uint64_t *tag, uint64_t *checksum, uint64_t *save_id);
uint64_t cache_hash(const void *p, size_t n, uint64_t seed);
}  // namespace lk

using lk::fail;
using lk::cache_identity;
using lk::cache_hash;

struct lkx_index {
    int centered = 0, store = 0, device = 0;
    int dim = 0;
    lk_index *dev = nullptr;
    std::vector<std::string> paths;
    std::unordered_map<std::string, int64_t> slot;
};

struct lkx_hits {
    std::vector<std::string> path;
    std::vector<float> score;
};

namespace {

int ensure_device(lkx_index *x, int len) {
    if (x->dev) return 0;
    if (len < 1) return fail(LK_EDIM, "embedindex: the first vector added fixes the dimension and must not be empty");
    LK_TRY(lk_index_create(len, x->store, x->centered, x->device, &x->dev));
    x->dim = len;
    return 0;
}

// A vector of the wrong length can never match (Cosine returns 0 on a length
// mismatch): it is kept as a zero row so that slot numbering stays dense.
const float *fit_row(const lkx_index *x, const float *vec, int len, std::vector<float> &tmp) {
    if (len == x->dim) return vec;
    tmp.assign((size_t)x->dim, 0.0f);
    return tmp.data();
}

// media-server/embedindex/embedindex.go:398-419; duplicates in `allow` collapse as in a Go set.
std::vector<int32_t> collect_slots(const lkx_index *x, const char *const *allow, int64_t n_allow) {
    std::vector<int32_t> slots;
    if (x->paths.empty() || n_allow <= 0) return slots;
    std::unordered_set<int64_t> seen;
    slots.reserve((size_t)std::min<int64_t>(n_allow, (int64_t)x->paths.size()));
    for (int64_t i = 0; i < n_allow; ++i) {
        if (!allow[i]) continue;
        auto it = x->slot.find(allow[i]);
        if (it == x->slot.end()) continue;
        if (seen.insert(it->second).second) slots.push_back((int32_t)it->second);
    }
    return slots;
}

// Device order is (score desc, slot asc); the reference orders equal scores by path.
lkx_hits *make_hits(const lkx_index *x, const int64_t *ids, const float *scores, int count) {
    lkx_hits *h = new lkx_hits();
    std::vector<int> order((size_t)count);
    for (int i = 0; i < count; ++i) order[i] = i;
    int i = 0;
    while (i < count) {
        int j = i + 1;
        while (j < count && scores[j] == scores[i]) ++j;
        if (j - i > 1)
            std::sort(order.begin() + i, order.begin() + j,
                      [&](int a, int b) { return x->paths[(size_t)ids[a]] < x->paths[(size_t)ids[b]]; });
        i = j;
    }
    h->path.reserve((size_t)count);
    h->score.reserve((size_t)count);
    for (int t = 0; t < count; ++t) {
        h->path.push_back(x->paths[(size_t)ids[order[t]]]);
        h->score.push_back(scores[order[t]]);
    }
    return h;
}

}  // namespace

extern "C" {

int lkx_new(int centered, int store, int device, lkx_index **out) {
    if (!out) return fail(LK_EINVAL, "lkx_new: out is NULL");
    *out = nullptr;
    if (store != LK_F32 && store != LK_F16 && store != LK_I8) return fail(LK_EINVAL, "lkx_new: unknown storage type");
    if (centered && store != LK_F32) return fail(LK_EINVAL, "lkx_new: centering needs float32 storage");
    if (lk_device_count() <= device || device < 0)
        return fail(LK_ECUDA, "lkx_new: no such CUDA device (this library has no CPU path)");
    lkx_index *x = new (std::nothrow) lkx_index();
    if (!x) return fail(LK_ENOMEM, "lkx_new: out of host memory");
    x->centered = centered ? 1 : 0;
    x->store = store;
    x->device = device;
    *out = x;
    return LK_OK;
}

int lkx_free(lkx_index *x) {
    if (!x) return LK_OK;
    if (x->dev) lk_index_destroy(x->dev);
    delete x;
    return LK_OK;
}

int lkx_add(lkx_index *x, const char *path, const float *vec, int len) {
    if (!x || !path || (len > 0 && !vec) || len < 0) return fail(LK_EINVAL, "lkx_add: bad argument");
    LK_TRY(ensure_device(x, len));
    std::vector<float> tmp;
    const float *row = fit_row(x, vec, len, tmp);
    auto it = x->slot.find(path);
    if (it != x->slot.end()) return lk_index_upsert_f32(x->dev, it->second, 1, row);  // in-place update
    const int64_t s = (int64_t)x->paths.size();
    LK_TRY(lk_index_upsert_f32(x->dev, s, 1, row));
    x->slot.emplace(path, s);
    x->paths.emplace_back(path);
    return LK_OK;
}

int lkx_add_batch(lkx_index *x, const char *const *paths, const float *rows, int64_t n, int len) {
    if (!x || n < 0 || (n > 0 && (!paths || !rows)) || len < 0) return fail(LK_EINVAL, "lkx_add_batch: bad argument");
    if (n == 0) return LK_OK;
    LK_TRY(ensure_device(x, len));
    if (len != x->dim) {
        for (int64_t i = 0; i < n; ++i) LK_TRY(lkx_add(x, paths[i], rows + (size_t)i * len, len));
        return LK_OK;
    }
    // Runs of new paths are appended with one upload; an existing (or repeated) path
    // ends the run so that every Add still takes effect in call order.
    int64_t run_start = 0;
    std::unordered_set<std::string> in_run;
    auto flush = [&](int64_t end) -> int {
        if (end <= run_start) return 0;
        const int64_t first = (int64_t)x->paths.size();
        LK_TRY(lk_index_upsert_f32(x->dev, first, end - run_start, rows + (size_t)run_start * len));
        for (int64_t i = run_start; i < end; ++i) {
            x->slot.emplace(paths[i], (int64_t)x->paths.size());
            x->paths.emplace_back(paths[i]);
        }
        in_run.clear();
        return 0;
    };
    for (int64_t i = 0; i < n; ++i) {
        if (!paths[i]) return fail(LK_EINVAL, "lkx_add_batch: NULL path");
        const bool known = x->slot.count(paths[i]) != 0 || in_run.count(paths[i]) != 0;
        if (known) {
            LK_TRY(flush(i));
            LK_TRY(lkx_add(x, paths[i], rows + (size_t)i * len, len));
            run_start = i + 1;
        } else {
            in_run.insert(paths[i]);
        }
    }
    return flush(n);
}

int lkx_delete(lkx_index *x, const char *path) {
    if (!x || !path) return fail(LK_EINVAL, "lkx_delete: bad argument");
    auto it = x->slot.find(path);
    if (it == x->slot.end()) return LK_OK;  // safe no-op
    const int64_t i = it->second, last = (int64_t)x->paths.size() - 1;
    LK_TRY(lk_index_swap_remove(x->dev, i));
    x->slot.erase(it);
    if (i != last) {
        x->paths[(size_t)i] = x->paths[(size_t)last];
        x->slot[x->paths[(size_t)i]] = i;
    }
    x->paths.pop_back();
    return LK_OK;
}

int64_t lkx_len(const lkx_index *x) { return x ? (int64_t)x->paths.size() : 0; }

lk_index *lkx_device_index(lkx_index *x) { return x ? x->dev : nullptr; }

int64_t lkx_slot_of(const lkx_index *x, const char *path) {
    if (!x || !path) return -1;
    auto it = x->slot.find(path);
    return it == x->slot.end() ? -1 : it->second;
}

int lkx_search_scored(lkx_index *x, const float *query, int len, int k, int has_allow, const char *const *allow,
                      int64_t n_allow, int scoring, lkx_hits **out) {
    if (!x || !out || (len > 0 && !query) || len < 0) return fail(LK_EINVAL, "lkx_search_scored: bad argument");
    *out = nullptr;
    if (!x->dev || x->paths.empty()) return LK_OK;  // n == 0 -> nil
    std::vector<int32_t> slots;
    if (has_allow) {
        slots = collect_slots(x, allow, n_allow);
        if (slots.empty()) return LK_OK;
    }
    if (k <= 0) return LK_OK;
    const int64_t n = has_allow ? (int64_t)slots.size() : (int64_t)x->paths.size();
    const int kk = (int)std::min<int64_t>(k, n);
    std::vector<float> tmp;
    const float *q = fit_row(x, query, len, tmp);  // wrong-length query: every Cosine is 0
    std::vector<int64_t> ids((size_t)kk);
    std::vector<float> scores((size_t)kk);
    int32_t count = 0;
    LK_TRY(lk_search(x->dev, q, 1, kk, scoring, has_allow ? slots.data() : nullptr, (int64_t)slots.size(),
                     ids.data(), scores.data(), nullptr, &count));
    *out = make_hits(x, ids.data(), scores.data(), count);
    return LK_OK;
}

int lkx_search_shared_scored(lkx_index *x, const float *const *pos, const int *pos_len, int npos, const float *posw,
                             int n_posw, const float *const *neg, const int *neg_len, int nneg, const float *negw,
                             int n_negw, int k, int has_allow, const char *const *allow, int64_t n_allow, int scoring,
                             lkx_hits **out) {
    if (!x || !out) return fail(LK_EINVAL, "lkx_search_shared_scored: bad argument");
    *out = nullptr;
    // embedvec.NewSharedQuery's validation, in its order (media-server/embedvec/shared.go:62-70, :89-109)
    if (npos <= 0) return fail(LK_EINVAL, "embedvec: shared query has no positive terms");
    if (n_posw != 0 && n_posw != npos)
        return fail(LK_EINVAL, "embedvec: shared query: " + std::to_string(npos) + " positives but " + std::to_string(n_posw) + " weights");
    if (nneg != n_negw)
        return fail(LK_EINVAL, "embedvec: shared query: " + std::to_string(nneg) + " negatives but " + std::to_string(n_negw) + " weights");
    const int d = pos_len[0];
    for (int i = 0; i < npos; ++i) {
        if (pos_len[i] != d) return fail(LK_EINVAL, "embedvec: shared query length mismatch: " + std::to_string(pos_len[i]) + " vs " + std::to_string(d));
        if (n_posw && !(posw[i] > 0)) return fail(LK_EINVAL, "embedvec: shared query positive weight must be > 0");
    }
    for (int i = 0; i < nneg; ++i)
        if (neg_len[i] != d) return fail(LK_EINVAL, "embedvec: shared query length mismatch: " + std::to_string(neg_len[i]) + " vs " + std::to_string(d));
    if (!x->dev || x->paths.empty()) return LK_OK;
    std::vector<int32_t> slots;
    if (has_allow) {
        slots = collect_slots(x, allow, n_allow);
        if (slots.empty()) return LK_OK;
    }
    if (k <= 0) return LK_OK;
    if (d != x->dim) return fail(LK_EDIM, "lkx_search_shared_scored: query vectors do not have the index's dimension");
    std::vector<float> P((size_t)npos * d), N((size_t)std::max(nneg, 1) * d);
    for (int i = 0; i < npos; ++i) std::copy(pos[i], pos[i] + d, P.begin() + (size_t)i * d);
    for (int i = 0; i < nneg; ++i) std::copy(neg[i], neg[i] + d, N.begin() + (size_t)i * d);
    const int64_t n = has_allow ? (int64_t)slots.size() : (int64_t)x->paths.size();
    const int kk = (int)std::min<int64_t>(k, n);
    std::vector<int64_t> ids((size_t)kk);
    std::vector<float> scores((size_t)kk);
    int32_t count = 0;
    LK_TRY(lk_search_shared(x->dev, P.data(), n_posw ? posw : nullptr, npos, nneg ? N.data() : nullptr,
                            nneg ? negw : nullptr, nneg, 0.25f /* DefaultSharedBeta */, 1.0f /* DefaultSharedLambda */,
                            kk, scoring, has_allow ? slots.data() : nullptr, (int64_t)slots.size(), ids.data(),
                            scores.data(), &count));
    *out = make_hits(x, ids.data(), scores.data(), count);
    return LK_OK;
}

int64_t lkx_hits_len(const lkx_hits *h) { return h ? (int64_t)h->path.size() : 0; }
const char *lkx_hits_path(const lkx_hits *h, int64_t i) {
    return (h && i >= 0 && i < (int64_t)h->path.size()) ? h->path[(size_t)i].c_str() : "";
}
float lkx_hits_score(const lkx_hits *h, int64_t i) {
    return (h && i >= 0 && i < (int64_t)h->score.size()) ? h->score[(size_t)i] : 0.0f;
}
void lkx_hits_free(lkx_hits *h) { delete h; }


// ---- on-disk cache: the device-side file of lk_index_save plus the paths in slot order ----

// `<path>.paths`: a 48-byte header (magic, the caller's tag, the checksum and the save number of the rows
// file it belongs to, the number of paths, a hash of everything behind the header), then per path a
// length and the bytes.
// A path table left over from another save of the same size, or one whose rows file was replaced, is
// refused: both files must come from the same lkx_save.
struct PathsHeader {
    char magic[8];  // "LKPTH001"
    uint64_t tag, rows_checksum, rows_save_id, n, body_hash;
};
static_assert(sizeof(PathsHeader) == 48, "paths header layout");

int lkx_save(lkx_index *x, const char *path, uint64_t tag) {
    if (!x || !path) return fail(LK_EINVAL, "lkx_save: bad argument");
    if (!x->dev) return fail(LK_EINVAL, "lkx_save: the index is empty");
    LK_TRY(lk_index_save(x->dev, path, tag));
    PathsHeader h;
    memcpy(h.magic, "LKPTH001", 8);
    uint64_t rows_tag = 0;
    LK_TRY(cache_identity(path, &rows_tag, &h.rows_checksum, &h.rows_save_id));
    h.tag = tag;
    h.n = x->paths.size();
    std::string body;
    for (const std::string &p : x->paths) {
        const uint32_t len = (uint32_t)p.size();
        body.append((const char *)&len, 4);
        body.append(p);
    }
    h.body_hash = cache_hash(body.data(), body.size(), h.rows_checksum);
    const std::string names = std::string(path) + ".paths", tmp = names + ".tmp";
    FILE *f = fopen(tmp.c_str(), "wb");
    if (!f) return fail(LK_EINVAL, "lkx_save: cannot create " + tmp);
    bool ok = fwrite(&h, sizeof(h), 1, f) == 1 && (body.empty() || fwrite(body.data(), 1, body.size(), f) == body.size());
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), names.c_str()) != 0) {
        remove(tmp.c_str());
        return fail(LK_EINVAL, "lkx_save: writing " + names + " failed");
    }
    return LK_OK;
}

int lkx_load(const char *path, uint64_t tag, int device, lkx_index **out) {
    if (!path || !out) return fail(LK_EINVAL, "lkx_load: bad argument");
    *out = nullptr;
    // the path table first: it is small, and a mismatch spares the upload of the rows
    const std::string names = std::string(path) + ".paths";
    uint64_t rows_tag = 0, rows_checksum = 0, rows_save_id = 0;
    LK_TRY(cache_identity(path, &rows_tag, &rows_checksum, &rows_save_id));
    FILE *f = fopen(names.c_str(), "rb");
    PathsHeader h;
    bool ok = f != nullptr && fread(&h, sizeof(h), 1, f) == 1 && memcmp(h.magic, "LKPTH001", 8) == 0 && h.tag == tag &&
              rows_tag == tag && h.rows_checksum == rows_checksum && h.rows_save_id == rows_save_id && h.n <= 0xfffffff0ull;
    std::string body;
    if (ok) {
        char buf[1 << 16];
        size_t got;
        while ((got = fread(buf, 1, sizeof(buf), f)) > 0) body.append(buf, got);
        ok = cache_hash(body.data(), body.size(), h.rows_checksum) == h.body_hash;
    }
    if (f) fclose(f);
    if (!ok) return fail(LK_EINVAL, "lkx_load: " + names + " is missing, damaged, or does not belong to these cached rows");
    lk_index *dev = nullptr;
    LK_TRY(lk_index_load(path, tag, device, &dev));
    lkx_index *x = new (std::nothrow) lkx_index();
    if (!x) {
        lk_index_destroy(dev);
        return fail(LK_ENOMEM, "lkx_load: out of host memory");
    }
    x->dev = dev;
    x->dim = lk_index_dim(dev);
    x->device = device;
    lk_index_kind(dev, &x->store, &x->centered);
    ok = (int64_t)h.n == lk_index_len(dev);
    size_t at = 0;
    for (uint64_t i = 0; ok && i < h.n; ++i) {
        uint32_t len = 0;
        ok = at + 4 <= body.size();
        if (ok) memcpy(&len, body.data() + at, 4);
        at += 4;
        ok = ok && len < (1u << 20) && at + len <= body.size();
        if (ok) {
            std::string p(body.data() + at, len);
            at += len;
            ok = x->slot.emplace(p, (int64_t)i).second;  // a path can own one slot only
            x->paths.emplace_back(std::move(p));
        }
    }
    ok = ok && at == body.size();
    if (!ok) {
        lkx_free(x);
        return fail(LK_EINVAL, "lkx_load: " + names + " does not match the cached rows");
    }
    *out = x;
    return LK_OK;
}

}  // extern "C"
