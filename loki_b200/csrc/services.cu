// Entry points for the service layer's brute-force fallbacks: the loops the reference runs when
// no index is installed for a model, or when a face search is restricted to a set of media paths
// (media-server/tasks/embed_task.go:249-272, media-server/tasks/face_search.go:199-216, :235-248).
// They score the vectors as the database holds them, un-normalised, with embedvec.CosineSim
// (media-server/embedvec/embedvec.go:127-141), so an index cannot stand in for them bit for bit;
// this is that loop on the device: upload the rows once, one fused scoring + top-k kernel.
#include <string>
#include <vector>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"
#include "scan.cuh"
#include "topk.cuh"

using namespace lk;

namespace {
struct Arena {
    unsigned char *p = nullptr;
    ~Arena() {
        if (p) cudaFree(p);
    }
};
}  // namespace

extern "C" int lk_cosine_sim_topk(const float *rows, int64_t n, int dim, const float *query, int k, const int32_t *allow_slots,
                                  int64_t n_allow, int device, int64_t *out_ids, float *out_scores, int32_t *out_count) {
    if (n < 0 || (n > 0 && !rows) || !query || dim < 1 || dim > LK_MAX_DIM || !out_count || (k > 0 && (!out_ids || !out_scores)))
        return fail(LK_EINVAL, "lk_cosine_sim_topk: bad argument");
    if (allow_slots == nullptr && n_allow > 0) return fail(LK_EINVAL, "lk_cosine_sim_topk: n_allow without allow_slots");
    *out_count = 0;
    const bool filtered = allow_slots != nullptr;
    const long long n_cand = filtered ? (long long)n_allow : (long long)n;
    if (filtered)
        for (int64_t i = 0; i < n_allow; ++i)
            if (allow_slots[i] < 0 || allow_slots[i] >= n) return fail(LK_EINVAL, "lk_cosine_sim_topk: allow slot out of range");
    if (k <= 0 || n_cand == 0) return LK_OK;
    if (n > 0x7ffffff0ll) return fail(LK_ERANGE, "lk_cosine_sim_topk: more than 2^31-16 rows");
    const long long k_eff = std::min<long long>(k, n_cand);
    const int passes = (int)((k_eff + kMaxK - 1) / kMaxK);  // kMaxK hits per pass; pass p accepts keys below pass p-1's last
    const int k_pass = (int)std::min<long long>(k_eff, kMaxK);
    if (lk_device_count() <= device || device < 0)
        return fail(LK_ECUDA, "lk_cosine_sim_topk: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    int sms = 0;
    LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    double q_n2 = 0.0;  // in element order, like the reference's loop
    for (int i = 0; i < dim; ++i) q_n2 += (double)query[i] * (double)query[i];

    ScanArgs a = {};
    a.n = n_cand;
    a.k = k_pass;
    int grid = 1;
    LK_TRY(cosine_sim_launch(a, dim, q_n2, sms, nullptr, &grid));
    // device: rows | query | slots | lists [grid][k] | ticket | keys, ids, scores, count
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += (size_t)round_up((int64_t)bytes, 256);
        return at;
    };
    const size_t o_rows = take((size_t)n * dim * 4), o_q = take((size_t)dim * 4), o_slots = take(filtered ? (size_t)n_cand * 4 : 4);
    const size_t o_part = take((size_t)grid * k_pass * 8), o_ticket = take(16), o_keys = take((size_t)k_eff * 8);
    const size_t o_ids = take((size_t)k_eff * 8), o_scores = take((size_t)k_eff * 4), o_count = take((size_t)passes * 4);
    Arena ar;
    {
        cudaError_t e = cudaMalloc((void **)&ar.p, off);
        if (e != cudaSuccess) return fail(LK_ENOMEM, std::string("lk_cosine_sim_topk: ") + cudaGetErrorString(e));
    }
    cudaStream_t st = nullptr;
    LK_CUDA(cudaMemcpyAsync(ar.p + o_rows, rows, (size_t)n * dim * 4, cudaMemcpyHostToDevice, st));
    LK_CUDA(cudaMemcpyAsync(ar.p + o_q, query, (size_t)dim * 4, cudaMemcpyHostToDevice, st));
    if (filtered) LK_CUDA(cudaMemcpyAsync(ar.p + o_slots, allow_slots, (size_t)n_cand * 4, cudaMemcpyHostToDevice, st));
    LK_CUDA(cudaMemsetAsync(ar.p + o_ticket, 0, 16, st));
    a.rows = ar.p + o_rows;
    a.ld = (long long)dim * 4;
    a.chunks = 0;
    a.slots = filtered ? (const int *)(ar.p + o_slots) : nullptr;
    a.query = ar.p + o_q;
    a.part = (unsigned long long *)(ar.p + o_part);
    a.ticket = (unsigned int *)(ar.p + o_ticket);
    a.out_iscores = nullptr;
    for (int p = 0; p < passes; ++p) {
        const long long done = (long long)p * kMaxK;
        a.k = (int)std::min<long long>(kMaxK, k_eff - done);
        unsigned long long *keys = (unsigned long long *)(ar.p + o_keys) + done;
        a.bound = p == 0 ? nullptr : keys - 1;
        a.out_keys = keys;
        a.out_ids = (long long *)(ar.p + o_ids) + done;
        a.out_scores = (float *)(ar.p + o_scores) + done;
        a.out_count = (int *)(ar.p + o_count) + p;
        LK_TRY(cosine_sim_launch(a, dim, q_n2, sms, st, nullptr));
    }
    std::vector<int> cnt((size_t)passes, 0);
    LK_CUDA(cudaMemcpyAsync(out_ids, ar.p + o_ids, (size_t)k_eff * 8, cudaMemcpyDeviceToHost, st));
    LK_CUDA(cudaMemcpyAsync(out_scores, ar.p + o_scores, (size_t)k_eff * 4, cudaMemcpyDeviceToHost, st));
    LK_CUDA(cudaMemcpyAsync(cnt.data(), ar.p + o_count, (size_t)passes * 4, cudaMemcpyDeviceToHost, st));
    LK_CUDA(cudaStreamSynchronize(st));
    long long total = 0;
    for (int p = 0; p < passes; ++p) total += cnt[p];
    for (long long i = total; i < k; ++i) {
        out_ids[i] = -1;
        out_scores[i] = 0.0f;
    }
    *out_count = (int32_t)total;
    return LK_OK;
}
