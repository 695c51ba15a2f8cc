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
    int qtile0, qtiles; // query tiles [qtile0, qtile0 + qtiles) are handled by this launch
    unsigned long long *cand;   // scratch [grid][128][1024] candidate keys
    unsigned long long *lists;  // out [slices][nq][k] ranked keys per corpus share
    int *error;
};

bool gemm_supported(long long ld, int k);
size_t gemm_cand_bytes(int grid);
int gemm_max_slices(int grid, int nq);   // lists a query can end up with
int gemm_launch(const unsigned char *d_rows, long long n, long long ld, const unsigned char *d_queries, int nq, int k,
                unsigned long long *d_cand, unsigned long long *d_lists, int *d_error, int sm_count,
                cudaStream_t stream, long long *launches);

}  // namespace lk
