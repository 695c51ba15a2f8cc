// Host-visible interface of the shared-concept scan (shared_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace lk {

// Scalar side of embedvec.SharedQuery (media-server/embedvec/shared.go:45-55), in device memory.
struct SharedParams {
    int m, rank, nneg;      // positives, basis vectors, negatives (m + rank + nneg <= 32)
    float gamma, lambda;
    float posw[32], posnorm[32], negw[32];
    float qb[256];          // m x rank
};

struct SharedArgs {
    const unsigned char *rows;
    long long ld;
    int chunks;
    long long n;
    const int *slots;
    const float *terms;          // [m + rank + nneg][ld/4] float32, zero padded (device)
    const SharedParams *params;  // device
    const float *cnorm;          // nullptr = plain; else per-slot centered norm
    const float *mu;             // [ld/4] mean vector, zero padded (centered only)
    int k;
    const unsigned long long *bound;
    const unsigned long long *floor;  // nullptr, or an exclusive lower bound for the keys (ScanArgs::floor)
    unsigned long long *part;
    int *part_cnt;               // nullptr, or [grid]: how many keys each CTA's list holds
    unsigned int *ticket;
    unsigned long long *out_keys;
    long long *out_ids;
    float *out_scores;
    int *out_iscores;
    int *out_count;
    long long shard_base;
};

// err: 0 ok, -1 the terms do not fit in shared memory, else a cudaError_t.
int shared_scan_grid(int terms, int chunks, int k, int device, int *err);
int shared_scan_launch(const SharedArgs &a, int terms, int grid, cudaStream_t stream);

// The float64 tensor-core kernel for whole-row scans (shared_mma.cu).
// shared_mma_launch: 0 = launched, 1 = not applicable (allow-list given, or nothing fits), else an error status.
bool shared_mma_fits(int terms, long long ld, int k);
int shared_mma_launch(const SharedArgs &a, int terms, int grid, cudaStream_t stream);

}  // namespace lk
