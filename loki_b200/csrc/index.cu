// C-ABI of the library (include/lokiscan.h): index storage in HBM, query
// preparation on the host, kernel launches, result marshalling.
//
// HBM layout of one index (all cudaMalloc'd, 256-byte aligned):
//   rows    capacity x ld bytes, row-major, ld = row bytes rounded up to 16 so
//           that every row starts on a 16-byte boundary (padding is zero)
//   scales  capacity x float   (int8 storage: per-row scale)
//   cnorm   capacity x float   (centered index: |row - mean|)
//   sum     dim x double, mu dim x float (centered index)
//   part    grid x k ranking keys + one ticket word: scratch of the scan kernel
//   result arena, query buffer, slot list, upload staging: grown on demand
#include <algorithm>
#include <atomic>
#include <chrono>
#include <unistd.h>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/lokiscan.h"
#include "build.cuh"
#include "comm.hpp"
#include <cstdio>

#include "gemm.cuh"
#include "multi.cuh"
#include "hostmath.hpp"
#include "index_internal.cuh"
#include "lk_common.cuh"
#include "scan.cuh"
#include "shared.cuh"
#include "topk.cuh"

namespace lk {

static thread_local std::string g_err;
void set_error(const std::string &msg) { g_err = msg; }
int fail(int status, const std::string &msg) {
    g_err = msg;
    return status;
}

}  // namespace lk

using namespace lk;

namespace lk {

static int use_device(const lk_index *idx) {
    LK_CUDA(cudaSetDevice(idx->device));
    return 0;
}

static int elem_bytes(int store) { return store == LK_F32 ? 4 : (store == LK_F16 ? 2 : 1); }

static int grow_rows(lk_index *idx, long long need) {
    if (need <= idx->cap) return 0;
    long long ncap = std::max<long long>(need, std::max<long long>(idx->cap * 2, 1024));
    unsigned char *nrows = nullptr;
    float *nscales = nullptr, *ncnorm = nullptr;
    cudaError_t e = cudaMalloc((void **)&nrows, (size_t)ncap * idx->ld);
    if (e == cudaSuccess && idx->store == LK_I8) e = cudaMalloc((void **)&nscales, (size_t)ncap * 4);
    if (e == cudaSuccess && idx->centered) e = cudaMalloc((void **)&ncnorm, (size_t)ncap * 4);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (nrows) cudaFree(nrows);
        if (nscales) cudaFree(nscales);
        if (ncnorm) cudaFree(ncnorm);
        return fail(LK_ENOMEM, std::string("growing the index to ") + std::to_string(ncap) + " rows: " + cudaGetErrorString(e));
    }
    if (idx->len > 0) {
        LK_CUDA(cudaMemcpyAsync(nrows, idx->d_rows, (size_t)idx->len * idx->ld, cudaMemcpyDeviceToDevice, idx->stream));
        if (nscales) LK_CUDA(cudaMemcpyAsync(nscales, idx->d_scales, (size_t)idx->len * 4, cudaMemcpyDeviceToDevice, idx->stream));
        if (ncnorm && idx->d_cnorm) LK_CUDA(cudaMemcpyAsync(ncnorm, idx->d_cnorm, (size_t)idx->len * 4, cudaMemcpyDeviceToDevice, idx->stream));
        LK_CUDA(cudaStreamSynchronize(idx->stream));
    }
    if (idx->d_rows) cudaFree(idx->d_rows);
    if (idx->d_scales) cudaFree(idx->d_scales);
    if (idx->d_cnorm) cudaFree(idx->d_cnorm);
    idx->d_rows = nrows;
    idx->d_scales = nscales;
    idx->d_cnorm = ncnorm;
    idx->cap = ncap;
    return 0;
}

// Add for n rows already on the device (media-server/embedindex/embedindex.go:176-194).
static int upsert_device(lk_index *idx, long long first, long long n, const float *d_src) {
    if (n == 0) return 0;
    LK_TRY(grow_rows(idx, first + n));
    const long long n_over = std::max<long long>(0, std::min(n, idx->len - first));
    unsigned char *dst = idx->d_rows + (size_t)first * idx->ld;
    if (idx->centered && n_over > 0) {
        LK_TRY(colsum_update_launch(dst, idx->ld, n_over, idx->dim, idx->d_sum, -1, idx->stream));
        idx->aux_launches++;
    }
    LK_TRY(normalize_store_launch(idx->store, d_src, n, idx->dim, dst, idx->ld,
                                  idx->d_scales ? idx->d_scales + first : nullptr, idx->sm_count, idx->stream));
    idx->aux_launches++;
    if (idx->centered) {
        LK_TRY(colsum_update_launch(dst, idx->ld, n, idx->dim, idx->d_sum, +1, idx->stream));
        idx->aux_launches++;
    }
    idx->len = std::max(idx->len, first + n);
    if (idx->center_live) {
        LK_TRY(centered_norm_launch(idx->d_rows, idx->ld, first, n, idx->dim, idx->d_mu, idx->mu_n2,
                                    idx->d_cnorm, idx->sm_count, idx->stream));
        idx->aux_launches++;
    }
    return 0;
}

// media-server/embedindex/embedindex.go:234-268
static int maybe_recenter(lk_index *idx) {
    if (!idx->centered) return 0;
    const long long n = idx->len;
    if (n < LK_MIN_CENTER_COUNT) {
        idx->center_live = false;
        idx->n_centered = n;
        return 0;
    }
    if (idx->center_live) {
        long long drift = n - idx->n_centered;
        if (drift < 0) drift = -drift;
        if (drift <= idx->n_centered / 10 + 32) return 0;
    }
    std::vector<double> sum((size_t)idx->dim);
    LK_CUDA(cudaMemcpyAsync(sum.data(), idx->d_sum, sizeof(double) * idx->dim, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    idx->h_mu.assign((size_t)idx->dim, 0.0f);
    idx->mu_n2 = hm::mean_from_sum(sum.data(), idx->dim, n, idx->h_mu.data());
    LK_CUDA(cudaMemcpyAsync(idx->d_mu, idx->h_mu.data(), sizeof(float) * idx->dim, cudaMemcpyHostToDevice, idx->stream));
    LK_TRY(centered_norm_launch(idx->d_rows, idx->ld, 0, n, idx->dim, idx->d_mu, idx->mu_n2, idx->d_cnorm,
                                idx->sm_count, idx->stream));
    idx->aux_launches++;
    LK_CUDA(cudaStreamSynchronize(idx->stream));  // h_mu is pageable: finish the copy before it can change
    idx->center_live = true;
    idx->n_centered = n;
    return 0;
}

// Normalise one raw query and convert it to what the scan kernel reads.
// Returns whether the query is scored centered.
constexpr int kFastWaitMs = 2500;  // longer than any bounded wait inside a kernel

static bool prepare_query(const lk_index *idx, const float *q, int scoring, unsigned char *dst,
                          float *cq, float *qscale) {
    const int d = idx->dim;
    std::vector<float> qn((size_t)d);
    hm::normalize(q, d, qn.data());
    memset(dst, 0, (size_t)idx->qbytes);
    *cq = 0.0f;
    *qscale = 0.0f;
    if (idx->store == LK_I8) {
        *qscale = hm::quantize_i8(qn.data(), d, reinterpret_cast<int8_t *>(dst));
        return false;
    }
    float *out = reinterpret_cast<float *>(dst);
    if (idx->store == LK_F32 && idx->center_live && scoring != LK_SCORE_PLAIN) {
        *cq = hm::center_query(qn.data(), idx->h_mu.data(), d, out);
        return true;
    }
    memcpy(out, qn.data(), sizeof(float) * (size_t)d);
    return false;
}

// the per-CTA list lengths live in the last bytes of the list scratch (room for 2,048 CTAs)
constexpr size_t kPartCntBytes = 8192;

static int ensure_scan_scratch(lk_index *idx, int k) {
    if (idx->grid_for_k != k) {
        LK_TRY(scan_plan(idx->type, idx->chunks, k, idx->device, &idx->plan));
        idx->grid = scan_max_grid(idx->plan);
        idx->grid_for_k = k;
    }
    LK_TRY(idx->part.reserve((size_t)idx->grid * k * 8 + kPartCntBytes));
    return 0;
}

// Enqueue the scan(s) of one prepared query.  k_eff hits are selected in passes of
// at most kMaxK; pass p accepts only keys below the last key of pass p-1.
// Arguments of one scan pass over this index (outputs and query are filled in by the caller).
static ScanArgs base_args(lk_index *idx, bool centered, float cq, float qscale, const int *d_slots,
                          long long n_cand, int k) {
    ScanArgs a;
    a.rows = idx->d_rows;
    a.ld = idx->ld;
    a.chunks = idx->chunks;
    a.n = n_cand;
    a.slots = d_slots;
    a.query = nullptr;
    a.cnorm = centered ? idx->d_cnorm : nullptr;
    a.cq = cq;
    a.k = k;
    a.bound = nullptr;
    a.floor = nullptr;
    a.floor_wait = 0;
    a.part = (unsigned long long *)idx->part.p;
    a.part_cnt = idx->part.p ? (int *)((unsigned char *)idx->part.p + idx->part.bytes - kPartCntBytes) : nullptr;
    a.ticket = idx->d_ticket;
    // consecutive launches may overlap at their edges: each uses its own batch counter and error word
    a.error = (int *)(idx->d_ticket + 8 + (idx->scan_launches % kScanOverlap));
    a.next_batch = idx->d_ticket + 2 + (idx->scan_launches % kScanOverlap);
    a.scales = idx->d_scales;
    a.qscale = qscale;
    a.shard_base = idx->shard_base;
    a.peer = nullptr;
    a.seq = 0;
    a.defer = 0;
    a.d_out_ids = nullptr;
    a.d_out_scores = nullptr;
    a.d_out_iscores = nullptr;
    a.d_out_count = nullptr;
    a.done_flag = nullptr;
    a.done_value = 0;
    return a;
}

// ---------------------------------------------------------------------------
// Large k: a sampled lower bound for the scan.
// Every CTA of a scan must keep its own best k rows, because all k best could sit in its
// part of the corpus; for k = 1,000 on 148 CTAs that is 148,000 keys kept, cut and merged to
// find 1,000.  Instead, a strided sample of S rows is scanned first (a gathered scan, a few
// microseconds); the sample's r-th best key becomes an exclusive lower bound for the real
// scan.  r is chosen so that k lies four standard deviations below the expected number of corpus
// rows above the bound (a few k): each CTA then keeps a few dozen keys.
// If fewer than k hits come out after all (a sample that misrepresents the corpus), the
// caller repeats the scan without the bound, so the result is exact either way.
// ---------------------------------------------------------------------------
constexpr int kFloorMinK = 256;       // below this the per-CTA lists are cheap anyway
constexpr int kSampleMin = 8192, kSampleMax = 32768;
constexpr int kFloorChunk = 64;       // queries of a batch whose sample scans are issued together, ahead of their scans

__global__ void k_fill_stride(int *slots, int n, long long len) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        slots[i] = (int)((long long)i * len / n);  // evenly spread over the rows
}

static bool floor_applies(const lk_index *idx, bool filtered, bool sharded, int k_eff, int passes) {
    return !idx->no_floor && !filtered && !sharded && passes == 1 && k_eff >= kFloorMinK &&
           idx->len >= 64ll * k_eff && idx->len >= 4ll * kSampleMin;
}

// Rows in the sample of the index as it stands, and the rank of the sample's key that serves as the bound.
static int sample_rows(const lk_index *idx, int k_eff) {
    // about 8 of the k best rows fall into the sample: the bound's rank then stays within 32, where a
    // scan keeps its candidates in registers and merges without a sort
    return (int)std::min<long long>(kSampleMax, std::max<long long>(kSampleMin, 8 * idx->len / k_eff)) & ~31;
}
static int sample_rank(const lk_index *idx, int k_eff, int S) {
    const double r = (double)k_eff * S / (double)idx->len;
    const double x = (4.0 + std::sqrt(16.0 + 4.0 * r)) * 0.5;  // r' - 4 sqrt(r') >= r
    return std::min<int>(kMaxK, std::max<int>(16, (int)std::ceil(x * x)));
}
// The sample's slots at the head of d_sample (of at least `bytes`), refilled when the buffer or the index changed.
static int sample_slots(lk_index *idx, int S, size_t bytes) {
    const void *before = idx->d_sample.p;
    LK_TRY(idx->d_sample.reserve(bytes));
    if (idx->d_sample.p != before || idx->sample_len != idx->len || idx->sample_n != S) {
        k_fill_stride<<<64, 256, 0, idx->stream>>>((int *)idx->d_sample.p, S, idx->len);
        LK_CUDA(cudaGetLastError());
        idx->sample_len = idx->len;
        idx->sample_n = S;
        idx->aux_launches++;
    }
    return 0;
}

// Enqueue the sample scan of one prepared query (in device memory, or inline in `inl`); *floor_out
// receives the device address of the bound.  A batch issues the sample scans of up to kFloorChunk
// queries first (`blocks` of them, this one writing output block `block`) and the real scans after
// them: the real scans then follow one another directly and overlap at their edges.
static int enqueue_sample_scan(lk_index *idx, const unsigned char *d_q, const unsigned char *inl, bool centered, float cq,
                               float qscale, int k_eff, const unsigned long long **floor_out, int block = 0, int blocks = 1) {
    const int S = sample_rows(idx, k_eff);
    const int rr = sample_rank(idx, k_eff, S);
    if (idx->plan_sample_k != rr) {
        LK_TRY(scan_plan(idx->type, idx->chunks, rr, idx->device, &idx->plan_sample));
        idx->plan_sample_k = rr;
    }
    // slots [S] | per block: keys [rr] | ids [rr] | scores [rr] | iscores [rr] | count
    const size_t block_bytes = (size_t)round_up((int64_t)rr * 24 + 16, 256);
    const size_t o_keys = (size_t)round_up((int64_t)S * 4, 256) + (size_t)block * block_bytes, o_ids = o_keys + (size_t)rr * 8;
    const size_t o_sc = o_ids + (size_t)rr * 8, o_isc = o_sc + (size_t)rr * 4, o_cnt = o_isc + (size_t)rr * 4;
    LK_TRY(sample_slots(idx, S, (size_t)round_up((int64_t)S * 4, 256) + (size_t)std::max(blocks, block + 1) * block_bytes));
    LK_TRY(idx->part.reserve((size_t)scan_max_grid(idx->plan_sample) * rr * 8 + kPartCntBytes));
    unsigned char *b = (unsigned char *)idx->d_sample.p;
    ScanArgs a = base_args(idx, centered, cq, qscale, (const int *)b, S, rr);
    a.query = d_q;
    if (d_q == nullptr) memcpy(a.query_inline, inl, (size_t)idx->qbytes);
    a.out_keys = (unsigned long long *)(b + o_keys);
    a.out_ids = (long long *)(b + o_ids);
    a.out_scores = (float *)(b + o_sc);
    a.out_iscores = (int *)(b + o_isc);
    a.out_count = (int *)(b + o_cnt);
    LK_TRY(scan_launch(idx->type, a, idx->plan_sample, idx->stream, false));
    idx->scan_launches++;
    *floor_out = (const unsigned long long *)(b + o_keys) + (rr - 1);
    return 0;
}

// Enqueue the scan(s) of one prepared query.  k_eff hits are selected in passes of
// at most kMaxK; pass p accepts only keys below the last key of pass p-1.
static int enqueue_query(lk_index *idx, const unsigned char *d_q, bool centered, float cq, float qscale,
                         const int *d_slots, long long n_cand, int k_eff, int k_stride, int passes,
                         const ResultArena &res, int qi, const PeerTable *peer = nullptr, unsigned int seq = 0,
                         int batch_pos = 0, const unsigned long long *floor = nullptr, bool floor_wait = false) {
    for (int p = 0; p < passes; ++p) {
        const int done = p * kMaxK;
        ScanArgs a = base_args(idx, centered, cq, qscale, d_slots, n_cand, std::min(kMaxK, k_eff - done));
        a.query = d_q;
        a.floor = floor;
        a.floor_wait = floor_wait ? 1 : 0;
        const size_t o = (size_t)qi * k_stride + done;
        a.bound = (p == 0) ? nullptr : res.d_keys() + o - 1;
        a.out_keys = res.d_keys() + o;
        a.out_ids = res.d_ids() + o;
        a.out_scores = res.d_scores() + o;
        a.out_iscores = res.d_iscores() + o;
        a.out_count = res.d_counts() + (size_t)qi * passes + p;
        a.peer = peer;
        a.seq = seq;
        if (peer) {  // queued sharded scans: this launch merges the query kPeerDefer places back in the batch
            a.defer = kPeerDefer;
            if (batch_pos >= kPeerDefer) {
                const size_t od = (size_t)(qi - kPeerDefer) * k_stride;
                a.d_out_ids = res.d_ids() + od;
                a.d_out_scores = res.d_scores() + od;
                a.d_out_iscores = res.d_iscores() + od;
                a.d_out_count = res.d_counts() + (size_t)(qi - kPeerDefer);
            }
        }
        LK_TRY(scan_launch(idx->type, a, idx->plan, idx->stream, scan_may_overlap(idx->plan, idx->scan_launches)));
        idx->scan_launches++;
    }
    return 0;
}

// After `count` queued sharded scans whose last query has index qi_last and sequence number
// seq_last: merge the queries that no later launch has merged.
static int drain_queued(lk_index *idx, const PeerTable *peer, const ResultArena &res, int qi_last, unsigned int seq_last,
                        int count, int k_eff) {
    const int m = std::min(count, kPeerDefer);
    if (m <= 0) return 0;
    DrainArgs d;
    d.peer = peer;
    d.seq_first = seq_last - (unsigned)(m - 1);
    d.count = m;
    d.k = k_eff;
    d.type = idx->type;
    const size_t o = (size_t)(qi_last - (m - 1)) * k_eff;
    d.out_ids = res.d_ids() + o;
    d.out_scores = res.d_scores() + o;
    d.out_iscores = res.d_iscores() + o;
    d.out_count = res.d_counts() + (qi_last - (m - 1));
    LK_TRY(peer_drain_launch(d, idx->stream));
    idx->aux_launches++;
    return 0;
}

static int unpack_results(const ResultArena &res, int nq, int k_user, int k_eff, int passes, int64_t *out_ids,
                          float *out_scores, int32_t *out_iscores, int32_t *out_counts);

// A batch of queries against an int8 index as one tensor-core matrix product with the
// top-k fused into its epilogue (gemm_i8.cu); same scores and ranking as query-by-query scans.
static int search_gemm(lk_index *idx, const float *queries, int nq, int k_user, int k_eff, int64_t *out_ids,
                       float *out_scores, int32_t *out_iscores, int32_t *out_counts) {
    const bool sharded = idx->comm != nullptr;
    const int slices = gemm_max_slices(idx->sm_count, nq, idx->len);
    const size_t e = (size_t)nq * k_eff;
    // device: queries | query scales | list bases (zeros) | shared thresholds (zeros) | lists [slices][nq][k] | merge scratch
    const size_t q_bytes = (size_t)round_up((int64_t)nq * idx->qbytes, 256);
    const size_t qs_bytes = (size_t)round_up((int64_t)nq * 4, 256);
    const size_t base_bytes = (size_t)round_up((int64_t)slices * 8, 256);
    const size_t thr_bytes = (size_t)round_up((int64_t)gemm_thr_bytes(nq), 256);
    const size_t list_bytes = (size_t)slices * e * 8;
    LK_TRY(idx->d_query.reserve(q_bytes + qs_bytes + base_bytes + thr_bytes + 2 * list_bytes));
    LK_TRY(idx->gemm_cand.reserve(gemm_cand_bytes(idx->sm_count)));
    LK_TRY(idx->res.shape(nq, k_eff, 1));
    // Queries are prepared on the device by the same kernel that stores rows (a query is
    // normalised and quantised exactly like a row): upload the raw float32 batch, convert.
    const size_t raw_bytes = (size_t)nq * idx->dim * sizeof(float);
    LK_TRY(idx->d_stage.reserve(raw_bytes));
    unsigned char *dq = (unsigned char *)idx->d_query.p;
    LK_CUDA(cudaMemcpyAsync(idx->d_stage.p, queries, raw_bytes, cudaMemcpyHostToDevice, idx->stream));
    LK_TRY(normalize_store_launch(LK_I8, (const float *)idx->d_stage.p, nq, idx->dim, dq, idx->ld,
                                  (float *)(dq + q_bytes), idx->sm_count, idx->stream));
    idx->aux_launches++;
    LK_CUDA(cudaMemsetAsync(dq + q_bytes + qs_bytes, 0, base_bytes + thr_bytes + list_bytes, idx->stream));
    unsigned long long *d_gthr = (unsigned long long *)(dq + q_bytes + qs_bytes + base_bytes);
    unsigned long long *d_lists = (unsigned long long *)(dq + q_bytes + qs_bytes + base_bytes + thr_bytes);
    int *d_err = (int *)(idx->d_ticket + 1);
    if (idx->len > 0)  // an empty shard contributes empty lists
        LK_TRY(gemm_launch(idx->d_rows, idx->len, idx->ld, dq, nq, k_eff, (unsigned long long *)idx->gemm_cand.p, d_gthr, d_lists,
                           d_err, idx->sm_count, idx->stream, &idx->aux_launches));
    MergeArgs m;
    m.keys = d_lists;
    m.payload = nullptr;
    m.qscales = (const float *)(dq + q_bytes);
    m.scales = idx->d_scales;
    m.scratch = d_lists + (size_t)slices * e;
    m.list_base = (const long long *)(dq + q_bytes + qs_bytes);
    m.lists = slices;
    m.nq = nq;
    m.k = k_eff;
    m.type = SCAN_I8;
    m.out_ids = idx->res.d_ids();
    m.out_scores = idx->res.d_scores();
    m.out_iscores = idx->res.d_iscores();
    m.out_count = idx->res.d_counts();
    m.out_keys = sharded ? idx->res.d_keys() : nullptr;
    LK_TRY(merge_launch(m, idx->stream));
    idx->aux_launches++;
    // sharded: ONE all-gather of every shard's nq x k ranked keys (+ finished scores), merged on every rank
    if (sharded) LK_TRY(comm_gather_merge(idx->comm, idx, idx->res, 0, nq, k_eff));
    int h_err = 0;
    LK_CUDA(cudaMemcpyAsync(idx->res.host.p, idx->res.dev.p, idx->res.copy_bytes, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaMemcpyAsync(&h_err, d_err, 4, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    if (h_err != 0) {
        LK_CUDA(cudaMemsetAsync(d_err, 0, 4, idx->stream));
        return fail(LK_ETIMEOUT, "the batched search kernel gave up on a bounded wait; results are not valid");
    }
    return unpack_results(idx->res, nq, k_user, k_eff, 1, out_ids, out_scores, out_iscores, out_counts);
}

// A batch of queries on a float32 index: 8 queries per pass over the corpus on the float64
// tensor-core path (multi_mma.cu), then one merge of the CTAs' lists per query.
static int search_multi_f32(lk_index *idx, const float *queries, int nq, int scoring, int k_user, int k_eff,
                            int64_t *out_ids, float *out_scores, int32_t *out_iscores, int32_t *out_counts) {
    const int grid = multi_grid(idx->len, idx->sm_count);
    const size_t e = (size_t)nq * k_eff;
    // device: prepared queries | cq | list bases (zeros) | lists [grid][nq][k] | merge scratch
    const size_t q_bytes = (size_t)round_up((int64_t)nq * idx->qbytes, 256);
    const size_t cq_bytes = (size_t)round_up((int64_t)nq * 4, 256);
    const size_t base_bytes = (size_t)round_up((int64_t)grid * 8, 256);
    const size_t list_bytes = (size_t)grid * e * 8;
    LK_TRY(idx->d_query.reserve(q_bytes + cq_bytes + base_bytes + 2 * list_bytes));
    LK_TRY(idx->h_query.reserve(q_bytes + cq_bytes));
    LK_TRY(idx->res.shape(nq, k_eff, 1));
    unsigned char *hq = (unsigned char *)idx->h_query.p;
    float *hcq = reinterpret_cast<float *>(hq + q_bytes);
    bool centered = false;
    for (int q = 0; q < nq; ++q) {
        float qscale = 0.0f;
        const bool c = prepare_query(idx, queries + (size_t)q * idx->dim, scoring, hq + (size_t)q * idx->qbytes, &hcq[q], &qscale);
        if (q == 0) centered = c;
    }
    unsigned char *dq = (unsigned char *)idx->d_query.p;
    LK_CUDA(cudaMemcpyAsync(dq, hq, q_bytes + cq_bytes, cudaMemcpyHostToDevice, idx->stream));
    LK_CUDA(cudaMemsetAsync(dq + q_bytes + cq_bytes, 0, base_bytes, idx->stream));
    unsigned long long *d_lists = (unsigned long long *)(dq + q_bytes + cq_bytes + base_bytes);
    int *d_err = (int *)(idx->d_ticket + 1);
    for (int q0 = 0; q0 < nq; q0 += kMultiQueries) {
        MultiArgs a;
        a.rows = idx->d_rows;
        a.ld = idx->ld;
        a.n = idx->len;
        a.queries = reinterpret_cast<const float *>(dq + (size_t)q0 * idx->qbytes);
        a.cq = reinterpret_cast<const float *>(dq + q_bytes) + q0;
        a.cnorm = centered ? idx->d_cnorm : nullptr;
        a.nq = std::min(kMultiQueries, nq - q0);
        a.q0 = q0;
        a.nq_total = nq;
        a.k = k_eff;
        a.lists = d_lists;
        a.error = d_err;
        LK_TRY(multi_launch(a, grid, idx->stream));
        idx->aux_launches++;
    }
    MergeArgs m;
    m.keys = d_lists;
    m.payload = nullptr;
    m.qscales = nullptr;
    m.scales = nullptr;
    m.scratch = d_lists + (size_t)grid * e;
    m.list_base = (const long long *)(dq + q_bytes + cq_bytes);
    m.lists = grid;
    m.nq = nq;
    m.k = k_eff;
    m.type = SCAN_F32;
    m.out_ids = idx->res.d_ids();
    m.out_scores = idx->res.d_scores();
    m.out_iscores = idx->res.d_iscores();
    m.out_count = idx->res.d_counts();
    m.out_keys = nullptr;
    LK_TRY(merge_launch(m, idx->stream));
    idx->aux_launches++;
    int h_err = 0;
    LK_CUDA(cudaMemcpyAsync(idx->res.host.p, idx->res.dev.p, idx->res.copy_bytes, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaMemcpyAsync(&h_err, d_err, 4, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    if (h_err != 0) {
        LK_CUDA(cudaMemsetAsync(d_err, 0, 4, idx->stream));
        return fail(LK_ETIMEOUT, "the batched search kernel gave up on a bounded wait; results are not valid");
    }
    return unpack_results(idx->res, nq, k_user, k_eff, 1, out_ids, out_scores, out_iscores, out_counts);
}

// Lowest-latency form of a single query: the prepared query rides in the launch
// parameters (no upload), the kernel writes the k results straight into mapped pinned
// host memory and releases a flag the host is polling (no download, no stream sync).
constexpr int kFastMaxK = 1024;
static int search_one_fast(lk_index *idx, const float *query, int scoring, const int *d_slots, long long n_cand,
                           int k_eff, const PeerTable *peer, int k_user, int64_t *out_ids, float *out_scores,
                           int32_t *out_iscores, int32_t *out_counts) {
    const size_t off_scores = (size_t)kFastMaxK * 8, off_iscores = off_scores + (size_t)kFastMaxK * 4;
    const size_t off_count = off_iscores + (size_t)kFastMaxK * 4, off_flag = off_count + 4;
    const void *zc_before = idx->zc.p;
    LK_TRY(idx->zc.reserve(off_flag + 4));
    if (idx->zc.p != zc_before) memset(idx->zc.p, 0, off_flag + 4);  // the flag must not start at a live value
    LK_TRY(idx->res.shape(1, k_eff, 1));  // device home of the ranked keys
    char *z = (char *)idx->zc.p;
    volatile unsigned int *flag = (volatile unsigned int *)(z + off_flag);
    float cq = 0.0f, qscale = 0.0f;
    ScanArgs a = base_args(idx, false, 0.0f, 0.0f, d_slots, n_cand, k_eff);
    const bool centered = prepare_query(idx, query, scoring, a.query_inline, &cq, &qscale);
    const bool use_floor = floor_applies(idx, d_slots != nullptr, peer != nullptr || idx->comm != nullptr, k_eff, 1);
    if (use_floor) {
        LK_TRY(enqueue_sample_scan(idx, nullptr, a.query_inline, centered, cq, qscale, k_eff, &a.floor));
        a.floor_wait = 1;
        a.part = (unsigned long long *)idx->part.p;  // the sample scan may have grown the scratch
        a.part_cnt = (int *)((unsigned char *)idx->part.p + idx->part.bytes - kPartCntBytes);
    }
    a.cnorm = centered ? idx->d_cnorm : nullptr;
    a.cq = cq;
    a.qscale = qscale;
    a.out_keys = idx->res.d_keys();
    a.out_ids = (long long *)z;
    a.out_scores = (float *)(z + off_scores);
    a.out_iscores = (int *)(z + off_iscores);
    a.out_count = (int *)(z + off_count);
    a.peer = peer;
    a.seq = peer ? comm_next_seq(idx->comm) : 0u;
    a.done_flag = (unsigned int *)(z + off_flag);
    a.done_value = ++idx->zc_seq ? idx->zc_seq : ++idx->zc_seq;  // never 0
    LK_TRY(scan_launch(idx->type, a, idx->plan, idx->stream, scan_may_overlap(idx->plan, idx->scan_launches)));
    idx->scan_launches++;
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned spins = 0; *flag != a.done_value; ++spins) {
        __builtin_ia32_pause();
        if ((spins & 0xfff) == 0xfff &&
            std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(kFastWaitMs)) {
            // not there yet: let the runtime tell whether the launch failed
            LK_CUDA(cudaStreamSynchronize(idx->stream));
            if (*flag != a.done_value) return fail(LK_ETIMEOUT, "lk_search: the scan finished without delivering its results");
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    int cnt = *(volatile int *)(z + off_count);
    if (cnt < 0) return fail(LK_ETIMEOUT, "a scan kernel gave up on a bounded wait (bulk copy or another rank); results are not valid");
    if (use_floor && cnt < k_eff) {  // the sampled bound was too high for this corpus: once more without it
        idx->no_floor = true;
        const int st = search_one_fast(idx, query, scoring, d_slots, n_cand, k_eff, peer, k_user, out_ids, out_scores, out_iscores,
                                       out_counts);
        idx->no_floor = false;
        return st;
    }
    if (cnt > k_eff) cnt = k_eff;
    const long long *ids = (const long long *)z;
    const float *sc = (const float *)(z + off_scores);
    const int *isc = (const int *)(z + off_iscores);
    for (int i = 0; i < k_user; ++i) {
        const bool hit = i < cnt;
        if (out_ids) out_ids[i] = hit ? (int64_t)ids[i] : -1;
        if (out_scores) out_scores[i] = hit ? sc[i] : 0.0f;
        if (out_iscores) out_iscores[i] = hit ? isc[i] : 0;
    }
    if (out_counts) out_counts[0] = cnt;
    return 0;
}

static int unpack_results(const ResultArena &res, int nq, int k_user, int k_eff, int passes,
                          int64_t *out_ids, float *out_scores, int32_t *out_iscores, int32_t *out_counts) {
    for (int q = 0; q < nq; ++q)
        for (int p = 0; p < passes; ++p)
            if (res.h_counts()[(size_t)q * passes + p] < 0)
                return fail(LK_ETIMEOUT, "a scan kernel gave up waiting for a bulk copy into shared memory; results are not valid");
    for (int q = 0; q < nq; ++q) {
        int cnt = 0;
        for (int p = 0; p < passes; ++p) cnt += res.h_counts()[(size_t)q * passes + p];
        if (cnt > k_eff) cnt = k_eff;
        const size_t so = (size_t)q * res.k, uo = (size_t)q * k_user;
        if (cnt == k_user) {  // the usual case: every place taken, whole rows move at once
            if (out_ids) memcpy(out_ids + uo, res.h_ids() + so, sizeof(int64_t) * (size_t)k_user);
            if (out_scores) memcpy(out_scores + uo, res.h_scores() + so, sizeof(float) * (size_t)k_user);
            if (out_iscores) memcpy(out_iscores + uo, res.h_iscores() + so, sizeof(int32_t) * (size_t)k_user);
            if (out_counts) out_counts[q] = cnt;
            continue;
        }
        for (int i = 0; i < k_user; ++i) {
            const bool hit = i < cnt;
            if (out_ids) out_ids[uo + i] = hit ? (int64_t)res.h_ids()[so + i] : -1;
            if (out_scores) out_scores[uo + i] = hit ? res.h_scores()[so + i] : 0.0f;
            if (out_iscores) out_iscores[uo + i] = hit ? res.h_iscores()[so + i] : 0;
        }
        if (out_counts) out_counts[q] = cnt;
    }
    return 0;
}

}  // namespace lk

// ===========================================================================
// C ABI
// ===========================================================================
extern "C" {

const char *lk_last_error(void) { return g_err.c_str(); }

const char *lk_version(void) { return "0.1.0"; }

int lk_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int lk_index_create(int dim, int store, int centered, int device, lk_index **out) {
    if (!out) return fail(LK_EINVAL, "lk_index_create: out is NULL");
    *out = nullptr;
    if (dim < 1 || dim > LK_MAX_DIM) return fail(LK_EDIM, "lk_index_create: dim out of range");
    if (store != LK_F32 && store != LK_F16 && store != LK_I8) return fail(LK_EINVAL, "lk_index_create: unknown storage type");
    if (centered && store != LK_F32) return fail(LK_EINVAL, "lk_index_create: centering needs float32 storage");
    if (lk_device_count() <= device || device < 0)
        return fail(LK_ECUDA, "lk_index_create: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    lk_index *idx = new (std::nothrow) lk_index();
    if (!idx) return fail(LK_ENOMEM, "lk_index_create: out of host memory");
    idx->dim = dim;
    idx->store = store;
    idx->centered = centered ? 1 : 0;
    idx->device = device;
    idx->type = store == LK_F32 ? SCAN_F32 : (store == LK_F16 ? SCAN_F16 : SCAN_I8);
    idx->ld = round_up((int64_t)dim * elem_bytes(store), 16);
    idx->chunks = (int)(idx->ld / 16);
    idx->qbytes = scan_query_bytes(idx->type, idx->ld);
    int st = 0;
    do {
        cudaError_t e = cudaStreamCreateWithFlags(&idx->stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreate(&idx->ev0);
        if (e == cudaSuccess) e = cudaEventCreate(&idx->ev1);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&idx->sm_count, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess) e = cudaMalloc((void **)&idx->d_ticket, 256);
        if (e == cudaSuccess) e = cudaMemsetAsync(idx->d_ticket, 0, 256, idx->stream);
        if (e == cudaSuccess && centered) {
            e = cudaMalloc((void **)&idx->d_sum, sizeof(double) * dim);
            if (e == cudaSuccess) e = cudaMemsetAsync(idx->d_sum, 0, sizeof(double) * dim, idx->stream);
            if (e == cudaSuccess) e = cudaMalloc((void **)&idx->d_mu, (size_t)idx->ld);
            if (e == cudaSuccess) e = cudaMemsetAsync(idx->d_mu, 0, (size_t)idx->ld, idx->stream);
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(idx->stream);
        if (e != cudaSuccess) st = fail(LK_ECUDA, std::string("lk_index_create: ") + cudaGetErrorString(e));
    } while (0);
    if (st != 0) {
        lk_index_destroy(idx);
        return st;
    }
    *out = idx;
    return LK_OK;
}

int lk_index_destroy(lk_index *idx) {
    if (!idx) return LK_OK;
    cudaSetDevice(idx->device);
    if (idx->stream) cudaStreamSynchronize(idx->stream);
    if (idx->d_rows) cudaFree(idx->d_rows);
    if (idx->d_scales) cudaFree(idx->d_scales);
    if (idx->d_cnorm) cudaFree(idx->d_cnorm);
    if (idx->d_sum) cudaFree(idx->d_sum);
    if (idx->d_mu) cudaFree(idx->d_mu);
    if (idx->d_ticket) cudaFree(idx->d_ticket);
    idx->part.release();
    idx->res.release();
    idx->d_query.release();
    idx->d_slots.release();
    idx->d_stage.release();
    idx->h_query.release();
    idx->zc.release();
    idx->gemm_cand.release();
    idx->d_sample.release();
    idx->gather.release();
    if (idx->ev0) cudaEventDestroy(idx->ev0);
    if (idx->ev1) cudaEventDestroy(idx->ev1);
    if (idx->stream) cudaStreamDestroy(idx->stream);
    cudaGetLastError();
    delete idx;
    return LK_OK;
}

int lk_index_reserve(lk_index *idx, int64_t n) {
    if (!idx || n < 0) return fail(LK_EINVAL, "lk_index_reserve: bad argument");
    LK_TRY(use_device(idx));
    return grow_rows(idx, n);
}

int64_t lk_index_len(const lk_index *idx) { return idx ? idx->len : 0; }
int lk_index_kind(const lk_index *idx, int *store, int *centered) {
    if (!idx) return fail(LK_EINVAL, "lk_index_kind: idx is NULL");
    if (store) *store = idx->store;
    if (centered) *centered = idx->centered;
    return LK_OK;
}
int lk_index_dim(const lk_index *idx) { return idx ? idx->dim : 0; }

int lk_index_upsert_f32_device(lk_index *idx, int64_t first_slot, int64_t n, const float *d_rows) {
    if (!idx || n < 0 || (n > 0 && !d_rows)) return fail(LK_EINVAL, "lk_index_upsert_f32_device: bad argument");
    if (first_slot < 0 || first_slot > idx->len) return fail(LK_EINVAL, "lk_index_upsert: first_slot must be within [0, len]");
    if (first_slot + n > 0xfffffff0ll) return fail(LK_ERANGE, "lk_index_upsert: more than 2^32-16 rows");
    LK_TRY(use_device(idx));
    LK_TRY(upsert_device(idx, first_slot, n, d_rows));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    return LK_OK;
}

int lk_index_upsert_f32(lk_index *idx, int64_t first_slot, int64_t n, const float *rows) {
    if (!idx || n < 0 || (n > 0 && !rows)) return fail(LK_EINVAL, "lk_index_upsert_f32: bad argument");
    if (first_slot < 0 || first_slot > idx->len) return fail(LK_EINVAL, "lk_index_upsert: first_slot must be within [0, len]");
    if (first_slot + n > 0xfffffff0ll) return fail(LK_ERANGE, "lk_index_upsert: more than 2^32-16 rows");
    LK_TRY(use_device(idx));
    LK_TRY(grow_rows(idx, first_slot + n));
    const size_t row_bytes = sizeof(float) * (size_t)idx->dim;
    const long long chunk_rows = std::max<long long>(1, (long long)((64u << 20) / row_bytes));
    LK_TRY(idx->d_stage.reserve((size_t)std::min<long long>(n, chunk_rows) * row_bytes));
    for (long long off = 0; off < n; off += chunk_rows) {
        const long long m = std::min(chunk_rows, n - off);
        LK_CUDA(cudaMemcpyAsync(idx->d_stage.p, rows + (size_t)off * idx->dim, (size_t)m * row_bytes,
                                cudaMemcpyHostToDevice, idx->stream));
        LK_TRY(upsert_device(idx, first_slot + off, m, (const float *)idx->d_stage.p));
        LK_CUDA(cudaStreamSynchronize(idx->stream));
    }
    return LK_OK;
}

int lk_index_swap_remove(lk_index *idx, int64_t slot) {
    if (!idx) return fail(LK_EINVAL, "lk_index_swap_remove: idx is NULL");
    if (slot < 0 || slot >= idx->len) return fail(LK_EINVAL, "lk_index_swap_remove: slot out of range");
    LK_TRY(use_device(idx));
    unsigned char *hole = idx->d_rows + (size_t)slot * idx->ld;
    if (idx->centered) {
        LK_TRY(colsum_update_launch(hole, idx->ld, 1, idx->dim, idx->d_sum, -1, idx->stream));
        idx->aux_launches++;
    }
    const long long last = idx->len - 1;
    if (slot != last) {
        LK_CUDA(cudaMemcpyAsync(hole, idx->d_rows + (size_t)last * idx->ld, (size_t)idx->ld, cudaMemcpyDeviceToDevice, idx->stream));
        if (idx->d_scales) LK_CUDA(cudaMemcpyAsync(idx->d_scales + slot, idx->d_scales + last, 4, cudaMemcpyDeviceToDevice, idx->stream));
        if (idx->d_cnorm && idx->center_live) LK_CUDA(cudaMemcpyAsync(idx->d_cnorm + slot, idx->d_cnorm + last, 4, cudaMemcpyDeviceToDevice, idx->stream));
    }
    idx->len = last;
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    return LK_OK;
}

int lk_index_read_rows(lk_index *idx, int64_t first, int64_t n, void *out, float *scales) {
    if (!idx || first < 0 || n < 0 || first + n > idx->len || (n > 0 && !out)) return fail(LK_EINVAL, "lk_index_read_rows: bad range");
    if (n == 0) return LK_OK;
    LK_TRY(use_device(idx));
    const size_t rb = (size_t)idx->dim * elem_bytes(idx->store);
    LK_CUDA(cudaMemcpy2DAsync(out, rb, idx->d_rows + (size_t)first * idx->ld, (size_t)idx->ld, rb, (size_t)n,
                              cudaMemcpyDeviceToHost, idx->stream));
    if (scales && idx->d_scales)
        LK_CUDA(cudaMemcpyAsync(scales, idx->d_scales + first, (size_t)n * 4, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    return LK_OK;
}

int lk_index_center_state(lk_index *idx, int *live, int64_t *n_centered, double *mu_n2, float *mu, double *sum, float *cnorm) {
    if (!idx) return fail(LK_EINVAL, "lk_index_center_state: idx is NULL");
    LK_TRY(use_device(idx));
    if (live) *live = idx->center_live ? 1 : 0;
    if (n_centered) *n_centered = idx->n_centered;
    if (mu_n2) *mu_n2 = idx->mu_n2;
    if (mu && idx->center_live) memcpy(mu, idx->h_mu.data(), sizeof(float) * (size_t)idx->dim);
    if (sum && idx->d_sum) LK_CUDA(cudaMemcpyAsync(sum, idx->d_sum, sizeof(double) * idx->dim, cudaMemcpyDeviceToHost, idx->stream));
    if (cnorm && idx->center_live && idx->len > 0)
        LK_CUDA(cudaMemcpyAsync(cnorm, idx->d_cnorm, sizeof(float) * (size_t)idx->len, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    return LK_OK;
}

int lk_search(lk_index *idx, const float *queries, int nq, int k, int scoring, const int32_t *allow_slots,
              int64_t n_allow, int64_t *out_ids, float *out_scores, int32_t *out_iscores, int32_t *out_counts) {
    if (!idx || nq < 0 || (nq > 0 && !queries)) return fail(LK_EINVAL, "lk_search: bad argument");
    if (allow_slots == nullptr && n_allow > 0) return fail(LK_EINVAL, "lk_search: n_allow without allow_slots");
    const auto t0 = std::chrono::steady_clock::now();
    LK_TRY(use_device(idx));
    LK_TRY(maybe_recenter(idx));
    const bool filtered = allow_slots != nullptr;
    const long long n_cand = filtered ? (long long)n_allow : idx->len;
    if (filtered)
        for (int64_t i = 0; i < n_allow; ++i)
            if (allow_slots[i] < 0 || allow_slots[i] >= idx->len) return fail(LK_EINVAL, "lk_search: allow slot out of range");
    auto no_hits = [&]() {
        for (int q = 0; q < nq; ++q) {
            if (out_counts) out_counts[q] = 0;
            for (int i = 0; i < std::max(k, 0); ++i) {
                if (out_ids) out_ids[(size_t)q * k + i] = -1;
                if (out_scores) out_scores[(size_t)q * k + i] = 0.0f;
                if (out_iscores) out_iscores[(size_t)q * k + i] = 0;
            }
        }
        return (int)LK_OK;
    };
    const bool sharded = idx->comm != nullptr;
    if (nq == 0 || k <= 0) return no_hits();
    if (n_cand == 0 && !sharded) return no_hits();
    // Per-shard k: a shard can contribute at most min(k, its candidates) hits, but with a
    // communicator every rank must run the same k so that the gathered lists line up.
    const int k_eff = sharded ? k : (int)std::min<long long>(k, n_cand);
    const int passes = (k_eff + kMaxK - 1) / kMaxK;
    if (sharded && passes > 1) return fail(LK_ERANGE, "lk_search: k above the single-pass limit is not supported on a sharded index");
    // (a sharded index takes the decision from what all ranks share: an empty or small shard must not
    // send one rank down another path than the others)
    if (idx->store == LK_I8 && nq >= GEMM_MIN_QUERIES && !filtered && gemm_supported(idx->ld, k_eff) &&
        (sharded || idx->len >= 4096) && !idx->no_gemm) {
        LK_TRY(search_gemm(idx, queries, nq, k, k_eff, out_ids, out_scores, out_iscores, out_counts));
        idx->last_search_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
        return LK_OK;
    }
    if (idx->store == LK_F32 && nq >= kMultiMinQueries && !filtered && !sharded && idx->len >= 8192 && !idx->no_gemm &&
        multi_supported(idx->ld, k_eff) && (long long)nq * k_eff <= (1 << 20)) {
        LK_TRY(search_multi_f32(idx, queries, nq, scoring, k, k_eff, out_ids, out_scores, out_iscores, out_counts));
        idx->last_search_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
        return LK_OK;
    }
    LK_TRY(ensure_scan_scratch(idx, std::min(k_eff, kMaxK)));
    const PeerTable *peer = sharded ? comm_peer_table(idx->comm, k_eff) : nullptr;
    if (nq == 1 && passes == 1 && k_eff <= kFastMaxK && idx->qbytes <= kInlineQueryBytes && (!sharded || peer)) {
        const int *d_sl = nullptr;
        if (filtered && n_cand > 0) {
            LK_TRY(idx->d_slots.reserve((size_t)n_cand * 4));
            LK_CUDA(cudaMemcpyAsync(idx->d_slots.p, allow_slots, (size_t)n_cand * 4, cudaMemcpyHostToDevice, idx->stream));
            d_sl = (const int *)idx->d_slots.p;
        }
        LK_TRY(search_one_fast(idx, queries, scoring, d_sl, n_cand, k_eff, peer, k, out_ids, out_scores, out_iscores,
                               out_counts));
        idx->last_search_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
        return LK_OK;
    }
    LK_TRY(idx->res.shape(nq, k_eff, passes));

    // queries: prepare on the host, one upload
    LK_TRY(idx->h_query.reserve((size_t)nq * idx->qbytes));
    LK_TRY(idx->d_query.reserve((size_t)nq * idx->qbytes));
    std::vector<float> cq((size_t)nq), qscale((size_t)nq);
    std::vector<char> cen((size_t)nq);
    for (int q = 0; q < nq; ++q)
        cen[q] = prepare_query(idx, queries + (size_t)q * idx->dim, scoring,
                               (unsigned char *)idx->h_query.p + (size_t)q * idx->qbytes, &cq[q], &qscale[q]);
    LK_CUDA(cudaMemcpyAsync(idx->d_query.p, idx->h_query.p, (size_t)nq * idx->qbytes, cudaMemcpyHostToDevice, idx->stream));
    const int *d_slots = nullptr;
    if (filtered && n_cand > 0) {
        LK_TRY(idx->d_slots.reserve((size_t)n_cand * 4));
        LK_CUDA(cudaMemcpyAsync(idx->d_slots.p, allow_slots, (size_t)n_cand * 4, cudaMemcpyHostToDevice, idx->stream));
        d_slots = (const int *)idx->d_slots.p;
    }
    // sharded: exchange inside the scan kernel over peer memory when that is set up, else NCCL
    unsigned int seq = 0;
    const bool use_floor = floor_applies(idx, filtered, sharded, k_eff, passes);
    const unsigned long long *floors[kFloorChunk] = {};
    for (int q = 0; q < nq; ++q) {
        const int c = q % kFloorChunk, chunk = std::min(kFloorChunk, nq - (q - c));
        if (use_floor && c == 0)  // the sample scans of the next chunk of queries, then their scans
            for (int j = 0; j < chunk; ++j)
                LK_TRY(enqueue_sample_scan(idx, (const unsigned char *)idx->d_query.p + (size_t)(q + j) * idx->qbytes, nullptr,
                                           cen[q + j] != 0, cq[q + j], qscale[q + j], k_eff, &floors[j], j, chunk));
        seq = peer ? comm_next_seq(idx->comm) : 0u;
        // only the chunk's last sample scan can still be running when a scan of the chunk starts
        LK_TRY(enqueue_query(idx, (const unsigned char *)idx->d_query.p + (size_t)q * idx->qbytes, cen[q] != 0, cq[q],
                             qscale[q], d_slots, n_cand, k_eff, k_eff, passes, idx->res, q, peer, seq, q,
                             use_floor ? floors[c] : nullptr, c == chunk - 1));
    }
    if (peer) LK_TRY(drain_queued(idx, peer, idx->res, nq - 1, seq, nq, k_eff));
    if (sharded && !peer) LK_TRY(comm_gather_merge(idx->comm, idx, idx->res, 0, nq, k_eff));
    LK_CUDA(cudaMemcpyAsync(idx->res.host.p, idx->res.dev.p, idx->res.copy_bytes, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    LK_TRY(unpack_results(idx->res, nq, k, k_eff, passes, out_ids, out_scores, out_iscores, out_counts));
    if (use_floor) {  // a query whose sampled bound turned out too high: once more, alone and without it
        std::vector<int32_t> counts((size_t)nq);
        for (int q = 0; q < nq; ++q) counts[q] = idx->res.h_counts()[q];
        for (int q = 0; q < nq; ++q) {
            if (counts[q] >= k_eff) continue;
            idx->no_floor = true;
            const int st = lk_search(idx, queries + (size_t)q * idx->dim, 1, k, scoring, nullptr, 0, out_ids ? out_ids + (size_t)q * k : nullptr,
                                     out_scores ? out_scores + (size_t)q * k : nullptr,
                                     out_iscores ? out_iscores + (size_t)q * k : nullptr, out_counts ? out_counts + q : nullptr);
            idx->no_floor = false;
            LK_TRY(st);
        }
    }
    idx->last_search_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return LK_OK;
}

int lk_search_shared(lk_index *idx, const float *pos, const float *posw, int npos, const float *neg, const float *negw,
                     int nneg, float beta, float lambda, int k, int scoring, const int32_t *allow_slots, int64_t n_allow,
                     int64_t *out_ids, float *out_scores, int32_t *out_count) {
    if (!idx || !out_count) return fail(LK_EINVAL, "lk_search_shared: bad argument");
    *out_count = 0;
    if (idx->store != LK_F32) return fail(LK_EINVAL, "lk_search_shared: needs float32 storage");
    if (idx->comm) return fail(LK_EINVAL, "lk_search_shared: not available on a sharded index");
    // constructor errors of embedvec.NewSharedQuery (media-server/embedvec/shared.go:62-70, :97-99)
    if (npos <= 0 || !pos) return fail(LK_EINVAL, "embedvec: shared query has no positive terms");
    if (nneg < 0 || (nneg > 0 && (!neg || !negw))) return fail(LK_EINVAL, "embedvec: shared query: negatives without weights");
    if (allow_slots == nullptr && n_allow > 0) return fail(LK_EINVAL, "lk_search_shared: n_allow without allow_slots");
    LK_TRY(use_device(idx));
    LK_TRY(maybe_recenter(idx));
    const bool centered = idx->center_live && scoring != LK_SCORE_PLAIN;
    hm::SharedPrep sp;
    const int pe = hm::shared_prepare(pos, posw, npos, neg, negw, nneg, idx->dim, beta, lambda,
                                      centered ? idx->h_mu.data() : nullptr, &sp);
    if (pe == 1) return fail(LK_EINVAL, "embedvec: shared query has no positive terms");
    if (pe == 2) return fail(LK_EINVAL, "embedvec: shared query positive weight must be > 0");
    const int T = sp.terms();
    if (T > LK_SHARED_MAX_TERMS || sp.m * sp.rank > 256) return fail(LK_ERANGE, "lk_search_shared: more than 32 query-side vectors");
    const bool filtered = allow_slots != nullptr;
    const long long n_cand = filtered ? (long long)n_allow : idx->len;
    if (filtered)
        for (int64_t i = 0; i < n_allow; ++i)
            if (allow_slots[i] < 0 || allow_slots[i] >= idx->len) return fail(LK_EINVAL, "lk_search_shared: allow slot out of range");
    if (n_cand == 0 || k <= 0) return LK_OK;
    const int k_eff = (int)std::min<long long>(k, n_cand);
    const int passes = (k_eff + kMaxK - 1) / kMaxK;
    const int k_pass = std::min(k_eff, kMaxK);
    int err = 0;
    const int grid = shared_scan_grid(T, idx->chunks, k_pass, idx->device, &err);
    if (err == -1) return fail(LK_ERANGE, "lk_search_shared: terms x dim too large for shared memory");
    if (err != 0 || grid <= 0) return fail(LK_ECUDA, std::string("shared scan occupancy query: ") + cudaGetErrorString((cudaError_t)err));
    LK_TRY(idx->part.reserve((size_t)grid * k_pass * 8 + kPartCntBytes));
    LK_TRY(idx->res.shape(1, k_eff, passes));
    // upload: terms padded to the row width, then the scalar block
    const size_t ldf = (size_t)idx->ld / 4;
    const size_t terms_bytes = (size_t)T * ldf * 4;
    const size_t par_off = (size_t)round_up((int64_t)terms_bytes, 16);
    LK_TRY(idx->h_query.reserve(par_off + sizeof(SharedParams)));
    LK_TRY(idx->d_query.reserve(par_off + sizeof(SharedParams)));
    unsigned char *hq = (unsigned char *)idx->h_query.p;
    memset(hq, 0, par_off + sizeof(SharedParams));
    for (int t = 0; t < T; ++t)
        memcpy(hq + (size_t)t * ldf * 4, &sp.vecs[(size_t)t * idx->dim], sizeof(float) * (size_t)idx->dim);
    SharedParams *hp = reinterpret_cast<SharedParams *>(hq + par_off);
    hp->m = sp.m;
    hp->rank = sp.rank;
    hp->nneg = sp.nneg;
    hp->gamma = sp.gamma;
    hp->lambda = sp.lambda;
    for (int i = 0; i < sp.m; ++i) {
        hp->posw[i] = sp.posw[i];
        hp->posnorm[i] = sp.posnorm[i];
    }
    for (int i = 0; i < sp.nneg; ++i) hp->negw[i] = sp.negw[i];
    for (int i = 0; i < sp.m * sp.rank; ++i) hp->qb[i] = sp.qb[i];
    LK_CUDA(cudaMemcpyAsync(idx->d_query.p, hq, par_off + sizeof(SharedParams), cudaMemcpyHostToDevice, idx->stream));
    const int *d_slots = nullptr;
    if (filtered) {
        LK_TRY(idx->d_slots.reserve((size_t)n_cand * 4));
        LK_CUDA(cudaMemcpyAsync(idx->d_slots.p, allow_slots, (size_t)n_cand * 4, cudaMemcpyHostToDevice, idx->stream));
        d_slots = (const int *)idx->d_slots.p;
    }
    // Large k: a sample scan first, whose r-th best key bounds the scan from below (see enqueue_sample_scan;
    // the same sample slots, the gathered kernel for the sample, plain stream order between the two launches).
    const bool use_floor = floor_applies(idx, filtered, false, k_eff, passes);
    const unsigned long long *floor = nullptr;
    if (use_floor) {
        const int S = sample_rows(idx, k_eff);
        const int rr = sample_rank(idx, k_eff, S);
        int serr = 0;
        const int sgrid = shared_scan_grid(T, idx->chunks, rr, idx->device, &serr);
        if (serr != 0 || sgrid <= 0) return fail(LK_ECUDA, "shared scan occupancy query (sample)");
        LK_TRY(idx->part.reserve((size_t)std::max(grid * k_pass, sgrid * rr) * 8 + kPartCntBytes));
        const size_t o_keys = (size_t)round_up((int64_t)S * 4, 256), o_ids = o_keys + (size_t)rr * 8, o_sc = o_ids + (size_t)rr * 8;
        const size_t o_cnt = o_sc + (size_t)rr * 4;
        LK_TRY(sample_slots(idx, S, o_cnt + 16));
        unsigned char *b = (unsigned char *)idx->d_sample.p;
        SharedArgs sa;
        sa.rows = idx->d_rows;
        sa.ld = idx->ld;
        sa.chunks = idx->chunks;
        sa.n = S;
        sa.slots = (const int *)b;
        sa.terms = (const float *)idx->d_query.p;
        sa.params = (const SharedParams *)((const unsigned char *)idx->d_query.p + par_off);
        sa.cnorm = centered ? idx->d_cnorm : nullptr;
        sa.mu = idx->d_mu;
        sa.k = rr;
        sa.bound = nullptr;
        sa.floor = nullptr;
        sa.part = (unsigned long long *)idx->part.p;
        sa.part_cnt = (int *)((unsigned char *)idx->part.p + idx->part.bytes - kPartCntBytes);
        sa.ticket = idx->d_ticket;
        sa.out_keys = (unsigned long long *)(b + o_keys);
        sa.out_ids = (long long *)(b + o_ids);
        sa.out_scores = (float *)(b + o_sc);
        sa.out_iscores = nullptr;
        sa.out_count = (int *)(b + o_cnt);
        sa.shard_base = idx->shard_base;
        LK_TRY(shared_scan_launch(sa, T, sgrid, idx->stream));
        idx->scan_launches++;
        floor = (const unsigned long long *)(b + o_keys) + (rr - 1);
    }
    for (int p = 0; p < passes; ++p) {
        const int done = p * kMaxK;
        SharedArgs a;
        a.rows = idx->d_rows;
        a.ld = idx->ld;
        a.chunks = idx->chunks;
        a.n = n_cand;
        a.slots = d_slots;
        a.terms = (const float *)idx->d_query.p;
        a.params = (const SharedParams *)((const unsigned char *)idx->d_query.p + par_off);
        a.cnorm = centered ? idx->d_cnorm : nullptr;
        a.mu = idx->d_mu;
        a.k = std::min(kMaxK, k_eff - done);
        a.bound = (p == 0) ? nullptr : idx->res.d_keys() + done - 1;
        a.floor = floor;
        a.part = (unsigned long long *)idx->part.p;
        a.part_cnt = (int *)((unsigned char *)idx->part.p + idx->part.bytes - kPartCntBytes);
        a.ticket = idx->d_ticket;
        a.out_keys = idx->res.d_keys() + done;
        a.out_ids = idx->res.d_ids() + done;
        a.out_scores = idx->res.d_scores() + done;
        a.out_iscores = idx->res.d_iscores() + done;
        a.out_count = idx->res.d_counts() + p;
        a.shard_base = idx->shard_base;
        LK_TRY(shared_scan_launch(a, T, grid, idx->stream));
        idx->scan_launches++;
    }
    LK_CUDA(cudaMemcpyAsync(idx->res.host.p, idx->res.dev.p, idx->res.copy_bytes, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    int32_t cnt = 0;
    LK_TRY(unpack_results(idx->res, 1, k, k_eff, passes, out_ids, out_scores, nullptr, &cnt));
    if (use_floor && cnt < k_eff) {  // the sampled bound was too high for this corpus: once more without it
        idx->no_floor = true;
        const int st = lk_search_shared(idx, pos, posw, npos, neg, negw, nneg, beta, lambda, k, scoring, allow_slots, n_allow,
                                        out_ids, out_scores, out_count);
        idx->no_floor = false;
        return st;
    }
    *out_count = cnt;
    return LK_OK;
}

// ---- device-resident queries ------------------------------------------------

int lk_queries_create(lk_index *idx, const float *queries, int nq, int scoring, lk_queries **out) {
    if (!idx || !out || nq <= 0 || !queries) return fail(LK_EINVAL, "lk_queries_create: bad argument");
    *out = nullptr;
    LK_TRY(use_device(idx));
    LK_TRY(maybe_recenter(idx));
    lk_queries *qs = new (std::nothrow) lk_queries();
    if (!qs) return fail(LK_ENOMEM, "lk_queries_create: out of host memory");
    qs->owner = idx;
    qs->nq = nq;
    qs->cq.resize((size_t)nq);
    qs->qscale.resize((size_t)nq);
    std::vector<unsigned char> host((size_t)nq * idx->qbytes);
    for (int q = 0; q < nq; ++q) {
        const bool c = prepare_query(idx, queries + (size_t)q * idx->dim, scoring, host.data() + (size_t)q * idx->qbytes,
                                     &qs->cq[q], &qs->qscale[q]);
        if (q == 0) qs->centered = c ? 1 : 0;
    }
    int st = qs->d_query.reserve(host.size());
    if (st == 0) {
        cudaError_t e = cudaMemcpy(qs->d_query.p, host.data(), host.size(), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) st = fail(LK_ECUDA, std::string("lk_queries_create: ") + cudaGetErrorString(e));
    }
    if (st != 0) {
        lk_queries_destroy(qs);
        return st;
    }
    *out = qs;
    return LK_OK;
}

int lk_queries_destroy(lk_queries *q) {
    if (!q) return LK_OK;
    if (q->owner) cudaSetDevice(q->owner->device);
    q->d_query.release();
    q->res.release();
    delete q;
    return LK_OK;
}

int lk_search_resident(lk_index *idx, lk_queries *q, int first, int count, int k) {
    if (!idx || !q || q->owner != idx || first < 0 || count < 0 || first + count > q->nq)
        return fail(LK_EINVAL, "lk_search_resident: bad argument");
    if (k <= 0 || k > kMaxK) return fail(LK_ERANGE, "lk_search_resident: k must be within 1..2048");
    LK_TRY(use_device(idx));
    const bool sharded = idx->comm != nullptr;
    if ((idx->len == 0 && !sharded) || count == 0) return LK_OK;
    const int k_eff = sharded ? k : (int)std::min<long long>(k, idx->len);
    LK_TRY(ensure_scan_scratch(idx, k_eff));
    if (q->res.nq != q->nq || q->res.k != k_eff) LK_TRY(q->res.shape(q->nq, k_eff, 1));
    const PeerTable *peer = sharded ? comm_peer_table(idx->comm, k_eff) : nullptr;
    unsigned int seq = 0;
    // large k: sampled floors, the queries that come out short are repeated without one by lk_queries_fetch
    const bool use_floor = floor_applies(idx, false, sharded, k_eff, 1);
    const unsigned long long *floors[kFloorChunk] = {};
    q->floored.resize((size_t)q->nq, 0);
    for (int i = first; i < first + count; ++i) {
        const int c = (i - first) % kFloorChunk, chunk = std::min(kFloorChunk, first + count - (i - c));
        if (use_floor && c == 0)
            for (int j = 0; j < chunk; ++j)
                LK_TRY(enqueue_sample_scan(idx, (const unsigned char *)q->d_query.p + (size_t)(i + j) * idx->qbytes, nullptr,
                                           q->centered != 0, q->cq[i + j], q->qscale[i + j], k_eff, &floors[j], j, chunk));
        q->floored[(size_t)i] = use_floor ? 1 : 0;
        seq = peer ? comm_next_seq(idx->comm) : 0u;
        LK_TRY(enqueue_query(idx, (const unsigned char *)q->d_query.p + (size_t)i * idx->qbytes, q->centered != 0,
                             q->cq[i], q->qscale[i], nullptr, idx->len, k_eff, k_eff, 1, q->res, i, peer, seq, i - first,
                             use_floor ? floors[c] : nullptr, c == chunk - 1));
        // one query at a time: without the peer path its candidates are gathered and merged here
        if (sharded && !peer) LK_TRY(comm_gather_merge(idx->comm, idx, q->res, i, 1, k_eff));
    }
    if (peer) LK_TRY(drain_queued(idx, peer, q->res, first + count - 1, seq, count, k_eff));
    return LK_OK;
}

int lk_queries_fetch(lk_index *idx, lk_queries *q, int first, int count, int k, int64_t *out_ids, float *out_scores,
                     int32_t *out_iscores, int32_t *out_counts) {
    if (!idx || !q || q->owner != idx || first < 0 || count < 0 || first + count > q->nq)
        return fail(LK_EINVAL, "lk_queries_fetch: bad argument");
    LK_TRY(use_device(idx));
    if (q->res.nq != q->nq || q->res.k <= 0) return fail(LK_EINVAL, "lk_queries_fetch: nothing has been searched yet");
    LK_CUDA(cudaMemcpyAsync(q->res.host.p, q->res.dev.p, q->res.copy_bytes, cudaMemcpyDeviceToHost, idx->stream));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    const ResultArena &r = q->res;
    // a query whose sampled floor turned out too high for this corpus came out short: once more without it
    int repeated = 0;
    for (int qi = first; qi < first + count && (size_t)qi < q->floored.size(); ++qi) {
        if (!q->floored[(size_t)qi]) continue;
        q->floored[(size_t)qi] = 0;
        if (r.h_counts()[qi] < 0 || r.h_counts()[qi] >= r.k) continue;
        if (repeated == 0) LK_TRY(ensure_scan_scratch(idx, r.k));  // (another search may have re-planned since)
        LK_TRY(enqueue_query(idx, (const unsigned char *)q->d_query.p + (size_t)qi * idx->qbytes, q->centered != 0, q->cq[qi],
                             q->qscale[qi], nullptr, idx->len, r.k, r.k, 1, q->res, qi));
        ++repeated;
    }
    if (repeated > 0) {
        LK_CUDA(cudaMemcpyAsync(q->res.host.p, q->res.dev.p, q->res.copy_bytes, cudaMemcpyDeviceToHost, idx->stream));
        LK_CUDA(cudaStreamSynchronize(idx->stream));
    }
    for (int i = 0; i < count; ++i) {
        const int qi = first + i;
        if (r.h_counts()[qi] < 0)
            return fail(LK_ETIMEOUT, "a scan kernel gave up waiting for a bulk copy into shared memory; results are not valid");
        int cnt = std::min(r.h_counts()[qi], r.k);
        for (int j = 0; j < k; ++j) {
            const bool hit = j < cnt;
            const size_t so = (size_t)qi * r.k + j, uo = (size_t)i * k + j;
            if (out_ids) out_ids[uo] = hit ? (int64_t)r.h_ids()[so] : -1;
            if (out_scores) out_scores[uo] = hit ? r.h_scores()[so] : 0.0f;
            if (out_iscores) out_iscores[uo] = hit ? r.h_iscores()[so] : 0;
        }
        if (out_counts) out_counts[i] = cnt;
    }
    return LK_OK;
}

int lk_timer_start(lk_index *idx) {
    if (!idx) return fail(LK_EINVAL, "lk_timer_start: idx is NULL");
    LK_TRY(use_device(idx));
    LK_CUDA(cudaEventRecord(idx->ev0, idx->stream));
    return LK_OK;
}

int lk_timer_stop(lk_index *idx, float *elapsed_ms) {
    if (!idx || !elapsed_ms) return fail(LK_EINVAL, "lk_timer_stop: bad argument");
    LK_TRY(use_device(idx));
    LK_CUDA(cudaEventRecord(idx->ev1, idx->stream));
    LK_CUDA(cudaEventSynchronize(idx->ev1));
    LK_CUDA(cudaEventElapsedTime(elapsed_ms, idx->ev0, idx->ev1));
    return LK_OK;
}

int lk_index_sync(lk_index *idx) {
    if (!idx) return fail(LK_EINVAL, "lk_index_sync: idx is NULL");
    LK_TRY(use_device(idx));
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    return LK_OK;
}

int lk_index_set_batch_mode(lk_index *idx, int mode) {
    if (!idx || (mode != 0 && mode != 1)) return fail(LK_EINVAL, "lk_index_set_batch_mode: bad argument");
    idx->no_gemm = (mode == 0);
    return LK_OK;
}

int lk_index_set_shard_base(lk_index *idx, int64_t shard_base) {
    if (!idx || shard_base < 0) return fail(LK_EINVAL, "lk_index_set_shard_base: bad argument");
    idx->shard_base = shard_base;
    return LK_OK;
}

int lk_stats(lk_index *idx, lk_stats_t *out) {
    if (!idx || !out) return fail(LK_EINVAL, "lk_stats: bad argument");
    out->len = idx->len;
    out->capacity = idx->cap;
    out->bytes_resident = (int64_t)idx->cap * idx->ld + (idx->d_scales ? idx->cap * 4 : 0) + (idx->d_cnorm ? idx->cap * 4 : 0) +
                          (int64_t)idx->part.bytes + (int64_t)idx->res.dev.bytes + (int64_t)idx->d_query.bytes +
                          (int64_t)idx->d_slots.bytes + (int64_t)idx->d_stage.bytes + (int64_t)idx->gather.bytes;
    out->scan_launches = idx->scan_launches;
    out->aux_launches = idx->aux_launches;
    out->last_search_ms = idx->last_search_ms;
    out->grid = idx->grid;
    out->sm_count = idx->sm_count;
    return LK_OK;
}

}  // extern "C"

// ---- on-disk cache of a built index ----------------------------------------------------
// The reference rebuilds its index from SQLite BLOBs at every start, one Add per row
// (media-server/tasks/embed_task.go:189-210, media-server/media/embedding.go:114-136); at
// millions of rows that rebuild dominates the time to the first query.  A built index is
// therefore written out as it sits in HBM (normalised / quantised rows, scales, centering
// state) and read back with plain copies.  The caller's tag (e.g. a hash of model name and
// row count) must match on load, as must a checksum of the payload.

namespace {

struct CacheHeader {  // 128 bytes, little-endian like the machine
    char magic[8];    // "LKIDX002"
    int32_t dim, store, centered, center_live;
    int64_t len, ld, n_centered;
    uint64_t tag, checksum;
    double mu_n2;
    uint64_t save_id;  // a number drawn at every save: what ties a path table to exactly this file
    unsigned char pad[48];
};
static_assert(sizeof(CacheHeader) == 128, "cache header layout");

// Word-wise FNV-1a-style hash over four interleaved lanes (the multiply's latency would
// otherwise cap one lane near 4 GB/s); sensitive to any flipped bit.  Chunks are multiples of
// 32 bytes except the last one of a region, whose tail goes through lane 0 byte by byte.
struct Hasher {
    uint64_t lane[4] = {0xcbf29ce484222325ull, 0x84222325cbf29ce4ull, 0x9ce484222325cbf2ull, 0x2325cbf29ce48422ull};
    void add(const void *p, size_t n) {
        const unsigned char *b = (const unsigned char *)p;
        size_t i = 0;
        uint64_t h0 = lane[0], h1 = lane[1], h2 = lane[2], h3 = lane[3];
        for (; i + 32 <= n; i += 32) {
            uint64_t w[4];
            memcpy(w, b + i, 32);
            h0 = (h0 ^ w[0]) * 0x100000001b3ull; h0 ^= h0 >> 29;
            h1 = (h1 ^ w[1]) * 0x100000001b3ull; h1 ^= h1 >> 29;
            h2 = (h2 ^ w[2]) * 0x100000001b3ull; h2 ^= h2 >> 29;
            h3 = (h3 ^ w[3]) * 0x100000001b3ull; h3 ^= h3 >> 29;
        }
        for (; i < n; ++i) h0 = (h0 ^ b[i]) * 0x100000001b3ull;
        lane[0] = h0; lane[1] = h1; lane[2] = h2; lane[3] = h3;
    }
    uint64_t value() const {
        uint64_t h = lane[0];
        for (int i = 1; i < 4; ++i) h = (h ^ lane[i]) * 0x100000001b3ull;
        return h;
    }
};

constexpr size_t kCacheChunk = 32u << 20;

// Two pinned buffers with an event each, so that the copy of one chunk overlaps the file
// I/O and hashing of the other.
struct CachePipe {
    lk::PinnedBuf buf[2];
    cudaEvent_t ev[2] = {nullptr, nullptr};
    int init() {
        for (int i = 0; i < 2; ++i) {
            LK_TRY(buf[i].reserve(kCacheChunk));
            LK_CUDA(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming));
        }
        return 0;
    }
    ~CachePipe() {
        for (int i = 0; i < 2; ++i) {
            buf[i].release();
            if (ev[i]) cudaEventDestroy(ev[i]);
        }
    }
};

// device -> file, hashing on the way: chunk i is written while chunk i + 1 is copied
int dump_device(lk_index *idx, const void *d, size_t bytes, FILE *f, CachePipe &pp, Hasher &hs) {
    const size_t n_chunks = (bytes + kCacheChunk - 1) / kCacheChunk;
    auto start = [&](size_t c) -> int {
        const size_t off = c * kCacheChunk, m = std::min(kCacheChunk, bytes - off);
        LK_CUDA(cudaMemcpyAsync(pp.buf[c & 1].p, (const unsigned char *)d + off, m, cudaMemcpyDeviceToHost, idx->stream));
        LK_CUDA(cudaEventRecord(pp.ev[c & 1], idx->stream));
        return 0;
    };
    if (n_chunks > 0) LK_TRY(start(0));
    for (size_t c = 0; c < n_chunks; ++c) {
        if (c + 1 < n_chunks) LK_TRY(start(c + 1));
        LK_CUDA(cudaEventSynchronize(pp.ev[c & 1]));
        const size_t m = std::min(kCacheChunk, bytes - c * kCacheChunk);
        hs.add(pp.buf[c & 1].p, m);
        if (fwrite(pp.buf[c & 1].p, 1, m, f) != m) return fail(LK_EINVAL, "lk_index_save: write failed");
    }
    return 0;
}
// file -> device: chunk i is uploaded while chunk i + 1 is read and hashed
int fill_device(lk_index *idx, void *d, size_t bytes, FILE *f, CachePipe &pp, Hasher &hs) {
    const size_t n_chunks = (bytes + kCacheChunk - 1) / kCacheChunk;
    bool used[2] = {false, false};
    for (size_t c = 0; c < n_chunks; ++c) {
        const int b = (int)(c & 1);
        if (used[b]) LK_CUDA(cudaEventSynchronize(pp.ev[b]));  // its previous upload has left the buffer
        const size_t off = c * kCacheChunk, m = std::min(kCacheChunk, bytes - off);
        if (fread(pp.buf[b].p, 1, m, f) != m) return fail(LK_EINVAL, "lk_index_load: the file is shorter than its header says");
        hs.add(pp.buf[b].p, m);
        LK_CUDA(cudaMemcpyAsync((unsigned char *)d + off, pp.buf[b].p, m, cudaMemcpyHostToDevice, idx->stream));
        LK_CUDA(cudaEventRecord(pp.ev[b], idx->stream));
        used[b] = true;
    }
    LK_CUDA(cudaStreamSynchronize(idx->stream));
    return 0;
}

}  // namespace

namespace lk {

// For the path table kept beside a cache file (host_index.cu): the tag and checksum in the header
// of the rows file, and the hash used for both files.
int cache_identity(const char *path, uint64_t *tag, uint64_t *checksum, uint64_t *save_id) {
    FILE *f = fopen(path, "rb");
    CacheHeader h;
    const bool ok = f != nullptr && fread(&h, 1, sizeof(h), f) == sizeof(h) && memcmp(h.magic, "LKIDX002", 8) == 0;
    if (f) fclose(f);
    if (!ok) return fail(LK_EINVAL, std::string("cannot read the cache header of ") + path);
    *tag = h.tag;
    *checksum = h.checksum;
    *save_id = h.save_id;
    return 0;
}
uint64_t cache_hash(const void *p, size_t n, uint64_t seed) {
    Hasher hs;
    hs.add(&seed, sizeof(seed));
    hs.add(p, n);
    return hs.value();
}

}  // namespace lk

extern "C" {

int lk_index_save(lk_index *idx, const char *path, uint64_t tag) {
    if (!idx || !path) return fail(LK_EINVAL, "lk_index_save: bad argument");
    if (idx->comm) return fail(LK_EINVAL, "lk_index_save: save each shard from its own unsharded handle");
    LK_TRY(use_device(idx));
    LK_TRY(maybe_recenter(idx));  // the cache holds the state a search would see
    const std::string tmp = std::string(path) + ".tmp";
    FILE *f = fopen(tmp.c_str(), "wb");
    if (!f) return fail(LK_EINVAL, std::string("lk_index_save: cannot create ") + tmp);
    CachePipe pin;
    int st = pin.init();
    CacheHeader h;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, "LKIDX002", 8);
    h.dim = idx->dim;
    h.store = idx->store;
    h.centered = idx->centered;
    h.center_live = idx->center_live ? 1 : 0;
    h.len = idx->len;
    h.ld = idx->ld;
    h.n_centered = idx->n_centered;
    h.tag = tag;
    h.mu_n2 = idx->mu_n2;
    h.save_id = (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count() * 0x9e3779b97f4a7c15ull ^
                (uint64_t)(uintptr_t)idx ^ ((uint64_t)getpid() << 32);
    Hasher hs;
    if (st == 0 && fwrite(&h, 1, sizeof(h), f) != sizeof(h)) st = fail(LK_EINVAL, "lk_index_save: write failed");
    if (st == 0 && idx->len > 0) st = dump_device(idx, idx->d_rows, (size_t)idx->len * idx->ld, f, pin, hs);
    if (st == 0 && idx->len > 0 && idx->d_scales) st = dump_device(idx, idx->d_scales, (size_t)idx->len * 4, f, pin, hs);
    if (st == 0 && idx->centered) {
        st = dump_device(idx, idx->d_sum, sizeof(double) * idx->dim, f, pin, hs);
        if (st == 0 && idx->center_live) {
            hs.add(idx->h_mu.data(), sizeof(float) * idx->dim);
            if (fwrite(idx->h_mu.data(), sizeof(float), (size_t)idx->dim, f) != (size_t)idx->dim)
                st = fail(LK_EINVAL, "lk_index_save: write failed");
            if (st == 0 && idx->len > 0) st = dump_device(idx, idx->d_cnorm, (size_t)idx->len * 4, f, pin, hs);
        }
    }
    if (st == 0) {
        hs.add(&h, sizeof(h));  // the header's own fields (checksum still zero) are covered too
        h.checksum = hs.value();
        if (fseek(f, 0, SEEK_SET) != 0 || fwrite(&h, 1, sizeof(h), f) != sizeof(h)) st = fail(LK_EINVAL, "lk_index_save: write failed");
    }
    if (fclose(f) != 0 && st == 0) st = fail(LK_EINVAL, "lk_index_save: close failed");
    if (st == 0 && rename(tmp.c_str(), path) != 0) st = fail(LK_EINVAL, std::string("lk_index_save: cannot rename to ") + path);
    if (st != 0) remove(tmp.c_str());
    return st;
}

int lk_index_load(const char *path, uint64_t tag, int device, lk_index **out) {
    if (!path || !out) return fail(LK_EINVAL, "lk_index_load: bad argument");
    *out = nullptr;
    FILE *f = fopen(path, "rb");
    if (!f) return fail(LK_EINVAL, std::string("lk_index_load: cannot open ") + path);
    CacheHeader h;
    int st = 0;
    if (fread(&h, 1, sizeof(h), f) != sizeof(h) || memcmp(h.magic, "LKIDX002", 8) != 0)
        st = fail(LK_EINVAL, "lk_index_load: not an index cache of this version");
    else if (h.tag != tag)
        st = fail(LK_EINVAL, "lk_index_load: the cache was written for another tag (model or row count changed)");
    else if (h.len < 0 || h.len > 0xfffffff0ll || h.dim < 1 || h.dim > LK_MAX_DIM)
        st = fail(LK_EINVAL, "lk_index_load: implausible header");
    lk_index *idx = nullptr;
    if (st == 0) st = lk_index_create(h.dim, h.store, h.centered, device, &idx);
    if (st == 0 && idx->ld != h.ld) st = fail(LK_EINVAL, "lk_index_load: row stride of the cache does not match this library");
    CachePipe pin;
    if (st == 0) st = pin.init();
    Hasher hs;
    if (st == 0 && h.len > 0) {
        st = grow_rows(idx, h.len);
        if (st == 0) st = fill_device(idx, idx->d_rows, (size_t)h.len * idx->ld, f, pin, hs);
        if (st == 0 && idx->d_scales) st = fill_device(idx, idx->d_scales, (size_t)h.len * 4, f, pin, hs);
    }
    if (st == 0 && idx->centered) {
        st = fill_device(idx, idx->d_sum, sizeof(double) * idx->dim, f, pin, hs);
        if (st == 0 && h.center_live) {
            idx->h_mu.assign((size_t)idx->dim, 0.0f);
            if (fread(idx->h_mu.data(), sizeof(float), (size_t)idx->dim, f) != (size_t)idx->dim)
                st = fail(LK_EINVAL, "lk_index_load: the file is shorter than its header says");
            if (st == 0) {
                hs.add(idx->h_mu.data(), sizeof(float) * idx->dim);
                cudaError_t e = cudaMemcpyAsync(idx->d_mu, idx->h_mu.data(), sizeof(float) * idx->dim, cudaMemcpyHostToDevice, idx->stream);
                if (e == cudaSuccess) e = cudaStreamSynchronize(idx->stream);
                if (e != cudaSuccess) st = fail(LK_ECUDA, std::string("lk_index_load: ") + cudaGetErrorString(e));
            }
            if (st == 0 && h.len > 0) st = fill_device(idx, idx->d_cnorm, (size_t)h.len * 4, f, pin, hs);
        }
    }
    if (st == 0 && fgetc(f) != EOF) st = fail(LK_EINVAL, "lk_index_load: the file is longer than its header says");
    if (st == 0) {
        CacheHeader plain = h;
        plain.checksum = 0;
        hs.add(&plain, sizeof(plain));
    }
    if (st == 0 && hs.value() != h.checksum) st = fail(LK_EINVAL, "lk_index_load: checksum mismatch, the cache is damaged");
    fclose(f);
    if (st != 0) {
        if (idx) lk_index_destroy(idx);
        return st;
    }
    idx->len = h.len;
    idx->center_live = h.center_live != 0;
    idx->n_centered = h.n_centered;
    idx->mu_n2 = h.mu_n2;
    *out = idx;
    return LK_OK;
}

}  // extern "C"
