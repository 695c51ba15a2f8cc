// Host-visible interface of the batched int8 tensor-core search (gemm_i8.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace lk {

constexpr int GEMM_MAX_K = 256;   // hits per query this path selects
constexpr int GEMM_MIN_QUERIES = 32;  // smaller batches run as single-query scans

struct GemmArgs {
    long long n;        // corpus rows
    int nq;             // queries
    int ks;             // 128-byte K slices per row
    int stages;         // corpus-tile stages in shared memory
    int k;
    int qtiles;         // 256-query tiles
    unsigned long long *cand;   // scratch (gemm_cand_bytes): candidate keys of every CTA's 128 queries
    unsigned long long *gthr;   // scratch (gemm_thr_bytes, zeroed): per query, the best k-th key any pair has reached
    unsigned long long *lists;  // out [slices][nq][k] ranked keys per corpus share
    int *error;
};

bool gemm_supported(long long ld, int k);
size_t gemm_cand_bytes(int sm_count);
size_t gemm_thr_bytes(int nq);
int gemm_max_slices(int sm_count, int nq, long long n);   // lists a query can end up with
int gemm_launch(const unsigned char *d_rows, long long n, long long ld, const unsigned char *d_queries, int nq, int k,
                unsigned long long *d_cand, unsigned long long *d_gthr, unsigned long long *d_lists, int *d_error,
                int sm_count, cudaStream_t stream, long long *launches);

}  // namespace lk
