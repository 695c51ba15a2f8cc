// Three-component PCA projection of an embedding cloud (the visualisation endpoint).
//
// Device replacement for embedvec.ProjectPCA3 (media-server/embedvec/pca.go:22-182): mean,
// power iteration with Gram-Schmidt deflation from a deterministic start vector, each
// iteration u = Xc^T (Xc v) with on-the-fly centering (covTimes, :130-182), projection of
// every point, one uniform scale into [-1, 1]^3, explained-variance fractions.
//
// Everything the reference computes in float64 is computed here in float64 with the same
// operations in the same order (multiply and add rounded separately, as Go does on amd64):
//   * a row's y_i = <x_i, v> is one thread walking the row left to right;
//   * u is accumulated per worker chunk of rows, one thread per column walking the chunk's
//     rows in order, and the chunks' partial sums are merged in chunk order, which is exactly
//     how covTimes orders its float64 additions for `workers` CPUs (the caller passes the
//     reference's runtime.NumCPU(); the component vectors depend on it in the last bits);
//   * the O(dim) vector steps (dot, orthogonalize, normalize) are sequential chains and run on
//     one thread, with the element-wise parts spread over the CTA.
// So coords are bit-identical to the reference's for the same `workers`.  The one exception is
// the total variance, a single 15-million-term chain in the reference: it is summed per row
// and then over rows, and the variance fractions agree to ~1e-13 relative instead of exactly.
//
// Bound: latency of the float64 add chains (the matrix, at most 20,000 x 1,024 floats in the
// reference's endpoint, stays in L2); a transposed copy makes the row-walking kernels coalesced.
#include <algorithm>
#include <string>
#include <vector>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"

namespace lk {

struct PcaState {
    double lambda;     // norm of u before normalisation in the last step
    double ysum;       // scratch of the merge
    double mv;         // <mean, v> for the next multiplication
    double total_var;
    unsigned long long max_abs_bits;  // largest |coordinate| seen, as the bits of a non-negative double
    int done;          // the current component has converged or died: further steps are no-ops
    int dead;          // lambda == 0: no variance left
    int n_comps;
};

__global__ void k_pca_transpose(const float *__restrict__ x, float *__restrict__ xt, int n, int d) {
    __shared__ float tile[32][33];
    const int i0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int i = i0 + r, j = j0 + threadIdx.x;
        tile[r][threadIdx.x] = (i < n && j < d) ? x[(size_t)i * d + j] : 0.0f;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int j = j0 + r, i = i0 + threadIdx.x;
        if (i < n && j < d) xt[(size_t)j * n + i] = tile[threadIdx.x][r];
    }
}

// mean[j] = (sum over rows, in row order, of float64(x[i][j])) / n       (pca.go:35-43)
__global__ void k_pca_mean(const float *__restrict__ x, int n, int d, double *__restrict__ mean) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= d) return;
    double s = 0.0;
    for (int i = 0; i < n; ++i) s = __dadd_rn(s, (double)x[(size_t)i * d + j]);
    mean[j] = s / (double)n;
}

// per-row sum of squared deviations (then summed over rows by k_pca_total)
__global__ void k_pca_rowvar(const float *__restrict__ xt, int n, int d, const double *__restrict__ mean,
                             double *__restrict__ rowvar) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    double s = 0.0;
    for (int j = 0; j < d; ++j) {
        const double dx = __dsub_rn((double)xt[(size_t)j * n + i], mean[j]);
        s = __dadd_rn(s, __dmul_rn(dx, dx));
    }
    rowvar[i] = s;
}
__global__ void k_pca_total(const double *__restrict__ rowvar, int n, PcaState *st) {
    double s = 0.0;
    for (int i = 0; i < n; ++i) s = __dadd_rn(s, rowvar[i]);
    st->total_var = s / (double)n;
}

// y_i = <x_i, v> - <mean, v>, one thread per row, left to right                (pca.go:159-164)
__global__ void k_pca_y(const float *__restrict__ xt, int n, int d, const double *__restrict__ v,
                        const PcaState *__restrict__ st, double *__restrict__ y) {
    if (st->done) return;
    extern __shared__ double sv[];
    for (int j = threadIdx.x; j < d; j += blockDim.x) sv[j] = v[j];
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    double s = 0.0;
    for (int j = 0; j < d; ++j) s = __dadd_rn(s, __dmul_rn((double)xt[(size_t)j * n + i], sv[j]));
    y[i] = __dsub_rn(s, st->mv);
}

// partial u of worker chunk w: u_w[j] = sum over the chunk's rows, in order, of y_i * x_ij;
// thread (w, 0) also sums the chunk's y                                      (pca.go:165-170)
__global__ void k_pca_u(const float *__restrict__ x, int n, int d, int chunk, const double *__restrict__ y,
                        const PcaState *__restrict__ st, double *__restrict__ part_u, double *__restrict__ part_y) {
    if (st->done) return;
    const int w = blockIdx.y, j = blockIdx.x * blockDim.x + threadIdx.x;
    const int lo = w * chunk, hi = min(n, lo + chunk);
    if (j < d) {
        double s = 0.0;
        for (int i = lo; i < hi; ++i) s = __dadd_rn(s, __dmul_rn(y[i], (double)x[(size_t)i * d + j]));
        part_u[(size_t)w * d + j] = s;
    }
    if (j == 0) {
        double s = 0.0;
        for (int i = lo; i < hi; ++i) s = __dadd_rn(s, y[i]);
        part_y[w] = s;
    }
}

__device__ double pca_dot_seq(const double *a, const double *b, int d) {  // pca.go:209-215
    double s = 0.0;
    for (int i = 0; i < d; ++i) s = __dadd_rn(s, __dmul_rn(a[i], b[i]));
    return s;
}

// One CTA.  mode 0: start of component c: v (uploaded start vector) is orthogonalised against
// the components found and normalised.  mode 1: end of a power-iteration step: merge the
// partials, finish u, orthogonalise, normalise, test convergence, v <- u.    (pca.go:60-80, :172-181)
__global__ void __launch_bounds__(256) k_pca_step(int mode, int d, int n_chunks, const double *__restrict__ mean,
                                                  const double *__restrict__ part_u, const double *__restrict__ part_y,
                                                  double *__restrict__ u, double *__restrict__ v,
                                                  const double *__restrict__ comps, PcaState *st) {
    __shared__ double s_p, s_norm;
    __shared__ int s_stop;
    const int tid = threadIdx.x;
    if (mode == 1 && st->done) return;
    double *t = (mode == 0) ? v : u;
    if (mode == 1) {
        if (tid == 0) {
            double ys = 0.0;
            for (int w = 0; w < n_chunks; ++w) ys = __dadd_rn(ys, part_y[w]);
            st->ysum = ys;
        }
        for (int j = tid; j < d; j += blockDim.x) {
            double s = 0.0;
            for (int w = 0; w < n_chunks; ++w) s = __dadd_rn(s, part_u[(size_t)w * d + j]);
            u[j] = s;
        }
        __syncthreads();
        const double ys = st->ysum;
        for (int j = tid; j < d; j += blockDim.x) u[j] = __dsub_rn(u[j], __dmul_rn(ys, mean[j]));
        __syncthreads();
    }
    const int nc = st->n_comps;
    for (int c = 0; c < nc; ++c) {  // orthogonalize (pca.go:198-206)
        if (tid == 0) s_p = pca_dot_seq(t, comps + (size_t)c * d, d);
        __syncthreads();
        const double p = s_p;
        for (int j = tid; j < d; j += blockDim.x) t[j] = __dsub_rn(t[j], __dmul_rn(p, comps[(size_t)c * d + j]));
        __syncthreads();
    }
    if (tid == 0) s_norm = sqrt(pca_dot_seq(t, t, d));  // normalize (pca.go:218-226)
    __syncthreads();
    const double nrm = s_norm;
    if (nrm != 0.0)
        for (int j = tid; j < d; j += blockDim.x) t[j] = t[j] / nrm;
    __syncthreads();
    if (tid == 0) {
        s_stop = 0;
        if (mode == 0) {
            st->lambda = 0.0;
            st->done = 0;
            st->dead = (nrm == 0.0) ? 1 : 0;
            if (nrm == 0.0) st->done = 1;
        } else {
            st->lambda = nrm;
            if (nrm == 0.0) {  // no variance left in the orthogonal complement
                st->dead = 1;
                st->done = 1;
                s_stop = 1;    // v keeps its value, as in the reference's early break
            } else if (fabs(pca_dot_seq(u, v, d)) > 1.0 - 1e-10) {
                st->done = 1;
            }
        }
    }
    __syncthreads();
    if (mode == 1 && !s_stop)
        for (int j = tid; j < d; j += blockDim.x) v[j] = u[j];
    __syncthreads();
    if (tid == 0) st->mv = pca_dot_seq(mean, v, d);
}

// coords[i][c] = float32(<x_i, comp_c> - <mean, comp_c>), and the largest |value|  (pca.go:90-106)
__global__ void k_pca_project(const float *__restrict__ xt, int n, int d, const double *__restrict__ comps, int n_comps,
                              const double *__restrict__ mean_dot, float *__restrict__ coords, PcaState *st) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    for (int c = 0; c < n_comps; ++c) {
        const double *comp = comps + (size_t)c * d;
        double s = 0.0;
        for (int j = 0; j < d; ++j) s = __dadd_rn(s, __dmul_rn((double)xt[(size_t)j * n + i], comp[j]));
        s = __dsub_rn(s, mean_dot[c]);
        coords[(size_t)i * 3 + c] = (float)s;
        atomicMax(&st->max_abs_bits, (unsigned long long)__double_as_longlong(fabs(s)));
    }
}
__global__ void k_pca_meandot(const double *__restrict__ mean, const double *__restrict__ comps, int d, int n_comps,
                              double *__restrict__ mean_dot) {
    if (threadIdx.x < n_comps) mean_dot[threadIdx.x] = pca_dot_seq(mean, comps + (size_t)threadIdx.x * d, d);
}
__global__ void k_pca_scale(float *__restrict__ coords, int n, const PcaState *__restrict__ st) {
    const double max_abs = __longlong_as_double((long long)st->max_abs_bits);
    if (!(max_abs > 0.0)) return;
    const float s = (float)(1.0 / max_abs);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * 3) coords[i] = __fmul_rn(coords[i], s);
}

struct PcaBufs {
    std::vector<void *> p;
    ~PcaBufs() {
        for (void *q : p) cudaFree(q);
    }
    template <typename T>
    cudaError_t alloc(T **out, size_t bytes) {
        void *q = nullptr;
        const cudaError_t e = cudaMalloc(&q, std::max<size_t>(bytes, 8));
        if (e == cudaSuccess) p.push_back(q);
        *out = (T *)q;
        return e;
    }
};

}  // namespace lk

using namespace lk;

extern "C" int lk_pca3(const float *vecs, int64_t n, int dim, int workers, int device, float *coords, double *variance) {
    if (n < 0 || dim < 0 || dim > LK_MAX_DIM || workers < 0 || !variance || (n > 0 && (!coords || (dim > 0 && !vecs))))
        return fail(LK_EINVAL, "lk_pca3: bad argument");
    if (n > 0x7fffffffll / 4) return fail(LK_ERANGE, "lk_pca3: too many vectors");
    variance[0] = variance[1] = variance[2] = 0.0;
    for (int64_t i = 0; i < n * 3; ++i) coords[i] = 0.0f;
    if (n == 0 || dim == 0) return LK_OK;
    if (lk_device_count() <= device || device < 0)
        return fail(LK_ECUDA, "lk_pca3: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    const int N = (int)n, d = dim;
    int w = workers > 0 ? workers : 1;
    if (w > N) w = N;
    const int chunk = (N + w - 1) / w, n_chunks = (N + chunk - 1) / chunk;  // pca.go:137-150
    PcaBufs B;
    float *d_x, *d_xt, *d_coords;
    double *d_mean, *d_rowvar, *d_y, *d_pu, *d_py, *d_u, *d_v, *d_comps, *d_md;
    PcaState *d_st;
    LK_CUDA(B.alloc(&d_x, (size_t)N * d * 4));
    LK_CUDA(B.alloc(&d_xt, (size_t)N * d * 4));
    LK_CUDA(B.alloc(&d_coords, (size_t)N * 3 * 4));
    LK_CUDA(B.alloc(&d_mean, (size_t)d * 8));
    LK_CUDA(B.alloc(&d_rowvar, (size_t)N * 8));
    LK_CUDA(B.alloc(&d_y, (size_t)N * 8));
    LK_CUDA(B.alloc(&d_pu, (size_t)n_chunks * d * 8));
    LK_CUDA(B.alloc(&d_py, (size_t)n_chunks * 8));
    LK_CUDA(B.alloc(&d_u, (size_t)d * 8));
    LK_CUDA(B.alloc(&d_v, (size_t)d * 8));
    LK_CUDA(B.alloc(&d_comps, (size_t)3 * d * 8));
    LK_CUDA(B.alloc(&d_md, 3 * 8));
    LK_CUDA(B.alloc(&d_st, sizeof(PcaState)));
    LK_CUDA(cudaMemcpy(d_x, vecs, (size_t)N * d * 4, cudaMemcpyHostToDevice));
    LK_CUDA(cudaMemset(d_st, 0, sizeof(PcaState)));
    LK_CUDA(cudaMemset(d_coords, 0, (size_t)N * 3 * 4));
    k_pca_transpose<<<dim3((N + 31) / 32, (d + 31) / 32), dim3(32, 8)>>>(d_x, d_xt, N, d);
    k_pca_mean<<<(d + 127) / 128, 128>>>(d_x, N, d, d_mean);
    k_pca_rowvar<<<(N + 127) / 128, 128>>>(d_xt, N, d, d_mean, d_rowvar);
    k_pca_total<<<1, 1>>>(d_rowvar, N, d_st);
    LK_CUDA(cudaGetLastError());
    PcaState h;
    LK_CUDA(cudaMemcpy(&h, d_st, sizeof(h), cudaMemcpyDeviceToHost));
    const double total_var = h.total_var;
    if (total_var == 0.0) return LK_OK;  // all points identical
    double eigen[3] = {0, 0, 0};
    int n_comps = 0;
    std::vector<double> start((size_t)d);
    for (int c = 0; c < 3; ++c) {
        // deterministicUnit (pca.go:187-195): a fixed LCG, integers and one exact division per element
        unsigned long long state = 0x9E3779B97F4A7C15ull + (unsigned long long)c * 0xBF58476D1CE4E5B9ull;
        for (int j = 0; j < d; ++j) {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            start[(size_t)j] = (double)(long long)(state >> 11) / (double)(1ull << 52) - 1.0;
        }
        LK_CUDA(cudaMemcpy(d_v, start.data(), (size_t)d * 8, cudaMemcpyHostToDevice));
        k_pca_step<<<1, 256>>>(0, d, n_chunks, d_mean, d_pu, d_py, d_u, d_v, d_comps, d_st);
        LK_CUDA(cudaGetLastError());
        LK_CUDA(cudaMemcpy(&h, d_st, sizeof(h), cudaMemcpyDeviceToHost));
        if (h.dead) break;  // the start vector lies in the span of the components found
        // up to 100 steps; converged or dead components turn the remaining launches into no-ops,
        // so the state is read back only every 10 steps
        for (int iter = 0; iter < 100 && !h.done; iter += 10) {
            for (int s = 0; s < 10; ++s) {
                k_pca_y<<<(N + 127) / 128, 128, (size_t)d * 8>>>(d_xt, N, d, d_v, d_st, d_y);
                k_pca_u<<<dim3((d + 127) / 128, n_chunks), 128>>>(d_x, N, d, chunk, d_y, d_st, d_pu, d_py);
                k_pca_step<<<1, 256>>>(1, d, n_chunks, d_mean, d_pu, d_py, d_u, d_v, d_comps, d_st);
            }
            LK_CUDA(cudaGetLastError());
            LK_CUDA(cudaMemcpy(&h, d_st, sizeof(h), cudaMemcpyDeviceToHost));
        }
        if (h.dead || h.lambda == 0.0) break;
        LK_CUDA(cudaMemcpy(d_comps + (size_t)n_comps * d, d_v, (size_t)d * 8, cudaMemcpyDeviceToDevice));
        eigen[n_comps] = h.lambda / (double)N;
        ++n_comps;
        h.n_comps = n_comps;
        h.done = 0;
        LK_CUDA(cudaMemcpy(d_st, &h, sizeof(h), cudaMemcpyHostToDevice));
    }
    if (n_comps > 0) {
        k_pca_meandot<<<1, 32>>>(d_mean, d_comps, d, n_comps, d_md);
        k_pca_project<<<(N + 127) / 128, 128>>>(d_xt, N, d, d_comps, n_comps, d_md, d_coords, d_st);
        k_pca_scale<<<(N * 3 + 255) / 256, 256>>>(d_coords, N, d_st);
        LK_CUDA(cudaGetLastError());
    }
    LK_CUDA(cudaMemcpy(coords, d_coords, (size_t)N * 3 * 4, cudaMemcpyDeviceToHost));
    for (int c = 0; c < n_comps; ++c) variance[c] = eigen[c] / total_var;
    return LK_OK;
}
