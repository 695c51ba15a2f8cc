// Corpus build kernels: normalise + convert rows on upload, and the centering state.
//
//   k_normalize_store   embedvec.Normalize (media-server/embedvec/embedvec.go:34-50) fused
//                       with the conversion to the storage type (float32 / half / int8+scale)
//   k_colsum_update     the float64 running column sum kept by Add/Delete
//                       (media-server/embedindex/embedindex.go:155-174)
//   k_centered_norm     centeredNorm for a range of rows
//                       (media-server/embedindex/embedindex.go:222-228, :260-266)
//
// Bit-exactness: the sum of squares and the column sum are accumulated in exactly
// the reference's order (element order within a row, slot order within a column),
// so the stored rows, the int8 codes and the mean vector equal what a CPU
// restatement of the Go code produces, bit for bit.  Only dot products that are
// reduced across lanes (k_centered_norm, the scan itself) differ in summation order.
#include <cuda_fp16.h>

#include "build.cuh"
#include "lk_common.cuh"

namespace lk {

// One warp per row.  Shared memory per warp: dim doubles (squares) + dim floats (the row) + ld bytes (packed output).
__global__ void __launch_bounds__(256) k_normalize_store(int type, const float *__restrict__ src, long long n,
                                                         int dim, unsigned char *__restrict__ dst, long long ld,
                                                         float *__restrict__ scales, int warps_per_cta) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp >= warps_per_cta) return;
    const size_t sq_bytes = (size_t)round_up((long long)dim * 8, 16);
    const size_t per_warp = sq_bytes + (size_t)round_up((long long)dim * 4, 16) + (size_t)ld;
    double *sq = reinterpret_cast<double *>(smem + per_warp * warp);
    float *x = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(sq) + sq_bytes);
    unsigned char *packed = reinterpret_cast<unsigned char *>(x) + round_up((long long)dim * 4, 16);

    for (long long row = (long long)blockIdx.x * warps_per_cta + warp; row < n;
         row += (long long)gridDim.x * warps_per_cta) {
        const float *s = src + row * dim;
        // All lanes widen their elements and square them (float32 squares are exact in
        // float64); one lane then adds the squares in element order.  Splitting it this way
        // keeps the conversions, which issue on a narrow pipe, off the one-lane chain.
        for (int i = lane; i < dim; i += 32) {
            const float f = s[i];
            x[i] = f;
            const double v = (double)f;
            sq[i] = v * v;
        }
        __syncwarp();
        double norm = 0.0;
        if (lane == 0) {
            double sum = 0.0;
            for (int i = 0; i < dim; ++i) sum = __dadd_rn(sum, sq[i]);
            norm = (sum == 0.0) ? 0.0 : sqrt(sum);
        }
        norm = __shfl_sync(0xffffffffu, norm, 0);
        float amax = 0.0f;
        if (norm != 0.0) {
            for (int i = lane; i < dim; i += 32) {
                const float y = (float)((double)x[i] / norm);
                x[i] = y;
                amax = fmaxf(amax, fabsf(y));
            }
        } else {
            // zero vector: stored unchanged
            for (int i = lane; i < dim; i += 32) amax = fmaxf(amax, fabsf(x[i]));
        }
        __syncwarp();
        unsigned char *out = dst + row * ld;
        if (type == 0) {  // float32
            float *o = reinterpret_cast<float *>(out);
            const int ldf = (int)(ld / 4);
            for (int i = lane; i < ldf; i += 32) o[i] = (i < dim) ? x[i] : 0.0f;
        } else if (type == 1) {  // half
            __half *o = reinterpret_cast<__half *>(packed);
            const int ldh = (int)(ld / 2);
            for (int i = lane; i < ldh; i += 32) o[i] = (i < dim) ? __float2half_rn(x[i]) : __float2half_rn(0.0f);
            __syncwarp();
            for (int j = lane; j < (int)(ld / 16); j += 32)
                reinterpret_cast<int4 *>(out)[j] = reinterpret_cast<const int4 *>(packed)[j];
        } else {  // int8 + scale
#pragma unroll
            for (int w = 16; w >= 1; w >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, w));
            const float scale = (amax == 0.0f) ? 0.0f : __fdiv_rn(amax, 127.0f);
            signed char *o = reinterpret_cast<signed char *>(packed);
            for (int i = lane; i < (int)ld; i += 32) {
                float r = 0.0f;
                if (i < dim && scale != 0.0f) {
                    r = rintf(__fdiv_rn(x[i], scale));  // round half to even
                    r = fminf(fmaxf(r, -127.0f), 127.0f);
                }
                o[i] = (signed char)(int)r;
            }
            __syncwarp();
            for (int j = lane; j < (int)(ld / 16); j += 32)
                reinterpret_cast<int4 *>(out)[j] = reinterpret_cast<const int4 *>(packed)[j];
            if (lane == 0) scales[row] = scale;
        }
        __syncwarp();
    }
}

// One thread per column; rows are visited in slot order so that the float64 sum
// rounds exactly as a row-by-row Add loop would.
__global__ void __launch_bounds__(128) k_colsum_update(const unsigned char *__restrict__ rows, long long ld,
                                                       long long n, int dim, double *__restrict__ sum, int sign) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= dim) return;
    double s = sum[d];
    const unsigned char *p = rows + (size_t)d * 4;
    long long i = 0;
    constexpr int U = 16;
    for (; i + U <= n; i += U) {
        float v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = *reinterpret_cast<const float *>(p + (i + u) * ld);
#pragma unroll
        for (int u = 0; u < U; ++u) s = (sign > 0) ? __dadd_rn(s, (double)v[u]) : __dsub_rn(s, (double)v[u]);
    }
    for (; i < n; ++i) {
        const float v = *reinterpret_cast<const float *>(p + i * ld);
        s = (sign > 0) ? __dadd_rn(s, (double)v) : __dsub_rn(s, (double)v);
    }
    sum[d] = s;
}

// One warp per row: cnorm = sqrt(max(0, 1 - 2*<v,mu> + |mu|^2)), <v,mu> rounded to float32 first.
__global__ void __launch_bounds__(256) k_centered_norm(const unsigned char *__restrict__ rows, long long ld,
                                                       long long first, long long n, int dim,
                                                       const float *__restrict__ mu, double mu_n2,
                                                       float *__restrict__ cnorm) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < n; r += nwarps) {
        const float *v = reinterpret_cast<const float *>(rows + (first + r) * ld);
        double acc = 0.0;
        for (int i = lane; i < dim; i += 32) acc = fma((double)v[i], (double)mu[i], acc);
#pragma unroll
        for (int w = 16; w >= 1; w >>= 1)
            acc += __longlong_as_double((long long)shfl_xor_u64((uint64_t)__double_as_longlong(acc), w));
        if (lane == 0) {
            const float c = (float)acc;
            double n2 = __dadd_rn(__dsub_rn(1.0, __dmul_rn(2.0, (double)c)), mu_n2);
            if (n2 < 0.0) n2 = 0.0;
            cnorm[first + r] = (float)sqrt(n2);
        }
    }
}

int normalize_store_launch(int type, const float *src, long long n, int dim, unsigned char *dst,
                           long long ld, float *scales, int sm_count, cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t per_warp = (size_t)round_up((long long)dim * 8, 16) + (size_t)round_up((long long)dim * 4, 16) + (size_t)ld;
    int warps = (int)((96 * 1024) / per_warp);
    if (warps > 8) warps = 8;
    if (warps < 1) warps = 1;
    const size_t smem = per_warp * warps;
    cudaError_t e = cudaFuncSetAttribute((const void *)k_normalize_store,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(4, std::string("normalize attr: ") + cudaGetErrorString(e));
    long long blocks = (n + warps - 1) / warps;
    const long long max_blocks = (long long)sm_count * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    k_normalize_store<<<(int)blocks, 256, smem, stream>>>(type, src, n, dim, dst, ld, scales, warps);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("normalize launch: ") + cudaGetErrorString(e));
    return 0;
}

int colsum_update_launch(const unsigned char *rows, long long ld, long long n, int dim, double *sum,
                         int sign, cudaStream_t stream) {
    if (n <= 0) return 0;
    k_colsum_update<<<(dim + 127) / 128, 128, 0, stream>>>(rows, ld, n, dim, sum, sign);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("colsum launch: ") + cudaGetErrorString(e));
    return 0;
}

int centered_norm_launch(const unsigned char *rows, long long ld, long long first, long long n, int dim,
                         const float *mu, double mu_n2, float *cnorm, int sm_count, cudaStream_t stream) {
    if (n <= 0) return 0;
    long long blocks = (n + 7) / 8;
    const long long max_blocks = (long long)sm_count * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    k_centered_norm<<<(int)blocks, 256, 0, stream>>>(rows, ld, first, n, dim, mu, mu_n2, cnorm);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("centered-norm launch: ") + cudaGetErrorString(e));
    return 0;
}

}  // namespace lk
