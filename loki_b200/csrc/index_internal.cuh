// Internal state behind the opaque handles of include/lokiscan.h.
#pragma once
#include <algorithm>
#include <string>
#include <vector>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"
#include "scan.cuh"

namespace lk {

// A device buffer that only grows.
struct DevBuf {
    void *p = nullptr;
    size_t bytes = 0;
    int reserve(size_t need) {
        if (need <= bytes) return 0;
        size_t nb = std::max(need, bytes * 2);
        nb = (size_t)round_up((int64_t)nb, 256);
        void *np = nullptr;
        cudaError_t e = cudaMalloc(&np, nb);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(LK_ENOMEM, std::string("cudaMalloc(") + std::to_string(nb) + "): " + cudaGetErrorString(e));
        }
        if (p) cudaFree(p);
        p = np;
        bytes = nb;
        return 0;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
};

struct PinnedBuf {
    void *p = nullptr;
    size_t bytes = 0;
    int reserve(size_t need) {
        if (need <= bytes) return 0;
        size_t nb = std::max(need, bytes * 2);
        void *np = nullptr;
        cudaError_t e = cudaMallocHost(&np, nb);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(LK_ENOMEM, std::string("cudaMallocHost: ") + cudaGetErrorString(e));
        }
        if (p) cudaFreeHost(p);
        p = np;
        bytes = nb;
        return 0;
    }
    void release() {
        if (p) cudaFreeHost(p);
        p = nullptr;
        bytes = 0;
    }
};

// Device-side results of nq queries x k hits, one contiguous arena so that a
// single copy brings everything back:  ids | scores | iscores | counts | keys
struct ResultArena {
    DevBuf dev;
    PinnedBuf host;
    int nq = 0, k = 0, passes = 1;
    size_t off_scores = 0, off_iscores = 0, off_counts = 0, off_keys = 0, copy_bytes = 0, total = 0;
    int shape(int nq_, int k_, int passes_) {
        nq = nq_;
        k = k_;
        passes = passes_;
        const size_t e = (size_t)nq * k;
        off_scores = e * 8;
        off_iscores = off_scores + e * 4;
        off_counts = off_iscores + e * 4;
        copy_bytes = (size_t)round_up((int64_t)(off_counts + (size_t)nq * passes * 4), 16);
        off_keys = copy_bytes;
        total = off_keys + e * 8;
        LK_TRY(dev.reserve(total));
        LK_TRY(host.reserve(copy_bytes));
        return 0;
    }
    long long *d_ids() const { return (long long *)dev.p; }
    float *d_scores() const { return (float *)((char *)dev.p + off_scores); }
    int *d_iscores() const { return (int *)((char *)dev.p + off_iscores); }
    int *d_counts() const { return (int *)((char *)dev.p + off_counts); }
    unsigned long long *d_keys() const { return (unsigned long long *)((char *)dev.p + off_keys); }
    const long long *h_ids() const { return (const long long *)host.p; }
    const float *h_scores() const { return (const float *)((char *)host.p + off_scores); }
    const int *h_iscores() const { return (const int *)((char *)host.p + off_iscores); }
    const int *h_counts() const { return (const int *)((char *)host.p + off_counts); }
    void release() {
        dev.release();
        host.release();
    }
};

// identity of a cache file written by lk_index_save, and the hash both cache files use (index.cu)
int cache_identity(const char *path, uint64_t *tag, uint64_t *checksum, uint64_t *save_id);
uint64_t cache_hash(const void *p, size_t n, uint64_t seed);

}  // namespace lk

struct lk_comm;

struct lk_index {
    int dim = 0, store = 0, centered = 0, device = 0;
    int type = 0;          // ScanType
    long long ld = 0;      // row stride in bytes
    int chunks = 0;
    int qbytes = 0;        // bytes of one prepared query in device memory
    long long len = 0, cap = 0;
    unsigned char *d_rows = nullptr;
    float *d_scales = nullptr;
    float *d_cnorm = nullptr;
    double *d_sum = nullptr;
    float *d_mu = nullptr;
    bool center_live = false;
    long long n_centered = 0;
    double mu_n2 = 0.0;
    std::vector<float> h_mu;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int sm_count = 0;
    // scan scratch
    lk::DevBuf part;
    unsigned int *d_ticket = nullptr;
    int grid_for_k = -1, grid = 0;
    lk::ScanPlan plan;
    // per-call buffers
    lk::ResultArena res;
    lk::DevBuf d_query, d_slots, d_stage;
    lk::PinnedBuf h_query;
    lk::PinnedBuf zc;           // mapped pinned block the kernel writes single-query results into
    unsigned int zc_seq = 0;
    // large-k searches: a strided sample of the rows is scanned first and gives the scan a lower bound
    lk::DevBuf d_sample;        // sample slot numbers | sample scan's outputs (keys, ids, scores, count)
    long long sample_len = -1;  // index length the slot numbers were made for
    int sample_n = 0;
    lk::ScanPlan plan_sample;
    int plan_sample_k = -1;
    bool no_floor = false;      // set while a search is repeated without the bound
    lk::DevBuf gemm_cand;       // candidate lists of the batched tensor-core search
    bool no_gemm = false;       // batches run as single-query scans (lk_index_set_batch_mode)
    // multi-GPU
    lk_comm *comm = nullptr;
    long long shard_base = 0;
    lk::DevBuf gather;  // all-gather receive buffer + merge scratch
    // stats
    long long scan_launches = 0, aux_launches = 0;
    float last_search_ms = 0.0f;
};

struct lk_queries {
    lk_index *owner = nullptr;
    int nq = 0;
    int centered = 0;
    lk::DevBuf d_query;
    std::vector<float> cq, qscale;
    std::vector<char> floored;  // queries scanned with a sampled floor and not fetched since
    lk::ResultArena res;
};

