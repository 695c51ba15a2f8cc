// Host-visible interface of the batched float32 scan (multi_mma.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace lk {

constexpr int kMultiQueries = 8;     // queries one launch scores together
constexpr int kMultiMaxK = 256;      // hits per query this path selects
constexpr int kMultiMinQueries = 3;  // smaller batches run as single-query scans

struct MultiArgs {
    const unsigned char *rows;  // corpus base (device), float32 rows
    long long ld;               // row stride in bytes
    long long n;                // rows
    const float *queries;       // [nq][ld / 4] prepared queries of this launch (device), zero padded
    const float *cq;            // [nq] <qc, mu> of each centered query (device)
    const float *cnorm;         // nullptr = plain cosine; else per-row centered norm
    int nq;                     // queries of this launch, 1..kMultiQueries
    int q0, nq_total;           // their place in the whole batch
    int k;
    unsigned long long *lists;  // out [grid][nq_total][k] ranked keys per CTA
    int *error;
};

bool multi_supported(long long ld, int k);
int multi_grid(long long n, int sm_count);
int multi_launch(const MultiArgs &a, int grid, cudaStream_t stream);

}  // namespace lk
