// Host-visible interface of the corpus build kernels (build_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace lk {

// type: 0 float32, 1 half, 2 int8 (+ scales).  src: n rows of dim floats (device).
int normalize_store_launch(int type, const float *src, long long n, int dim, unsigned char *dst,
                           long long ld, float *scales, int sm_count, cudaStream_t stream);
// sum[d] += sign * rows[i][d] for i = 0..n-1 in that order (float32 rows, ld bytes apart).
int colsum_update_launch(const unsigned char *rows, long long ld, long long n, int dim, double *sum,
                         int sign, cudaStream_t stream);
// cnorm[first + i] for i = 0..n-1.
int centered_norm_launch(const unsigned char *rows, long long ld, long long first, long long n, int dim,
                         const float *mu, double mu_n2, float *cnorm, int sm_count, cudaStream_t stream);

}  // namespace lk
