// All-pairs neighbour prescreen of face clustering: for every vector i the earlier
// vectors j < i whose float32 dot reaches a threshold, as ascending lists capped at 256.
//
// Device replacement for prescreenCandidates (media-server/tasks/face_cluster.go:1189-1285)
// and its scorer dotf (media-server/tasks/face_cluster.go:908-925).  This is the
// reference's other O(N^2 * dim) loop; it sits next to the scan path (it consumes the
// same float32 vectors) and is the first of the "next" rows around it.
//
// Arithmetic is dotf's, bit for bit: float32 multiply and add (never fused), four
// accumulators fed by element index mod 4 in ascending order, combined as
// (s0+s1)+(s2+s3); leftover elements of a length that is not a multiple of 4 go to s0.
// The reference scores most pairs through a four-row variant (dot4) whose summation
// order differs in the last bit; its own test defines the result by dotf
// (media-server/tasks/face_cluster_perf_test.go:52-81), and so does this kernel.
//
// Bound: float32 ALU (one multiply + one add per element pair, 2 N^2/2 dim operations);
// the vectors (N x dim x 4 B, e.g. 41 MB for 20,000 x 512) stay in L2.
#include <algorithm>
#include <string>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"

namespace lk {

constexpr int PT = 64;       // tile edge (rows and columns)
constexpr int PK = 16;       // elements of every vector staged per step
constexpr int PTHREADS = 256;
constexpr int PMAX = 256;    // maxFormCandidates (media-server/tasks/face_cluster.go:1156)

__device__ __forceinline__ void ptile_from_linear(long long t, int *bi, int *bj) {
    // lower triangle, row-major: row bi holds bi+1 tiles
    int r = (int)((sqrt(8.0 * (double)t + 1.0) - 1.0) * 0.5);
    while ((long long)r * (r + 1) / 2 > t) --r;
    while ((long long)(r + 1) * (r + 2) / 2 <= t) ++r;
    *bi = r;
    *bj = (int)(t - (long long)r * (r + 1) / 2);
}

__global__ void __launch_bounds__(PTHREADS) k_prescreen_pairs(const float *__restrict__ v, int n, int dim, int ld,
                                                              float threshold, long long n_tiles,
                                                              int *__restrict__ near, int *__restrict__ count) {
    // +4: rows lie 80 B = 5 x 16 B apart.  A thread's four columns are rows tx, tx+16, tx+32, tx+48 of Bs,
    // so the eight lanes of a quarter warp read eight neighbouring rows, which fall on eight different
    // 16-byte bank groups (four neighbouring rows per thread would put them on two).
    // Two copies of each tile: while the threads compute on one, the next step's floats go into the other,
    // which leaves one barrier per step.
    __shared__ float As[2][PT][PK + 4], Bs[2][PT][PK + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int dim4 = dim & ~3;
    for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        int bi, bj;
        ptile_from_linear(t, &bi, &bj);
        const int i0 = bi * PT, j0 = bj * PT;
        float acc[4][4][4];  // [row][col][accumulator]
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int m = 0; m < 4; ++m) acc[r][c][m] = 0.0f;
        // this thread's 4 floats of the staging step (zero past the end of a row or of the matrix):
        // fetched one step ahead, so the L2 latency hides behind the arithmetic of the step before
        const int lrow = tid >> 2, lkk = (tid & 3) * 4;
        const float *ap = (i0 + lrow < n) ? v + (size_t)(i0 + lrow) * ld + lkk : nullptr;
        const float *bp = (j0 + lrow < n) ? v + (size_t)(j0 + lrow) * ld + lkk : nullptr;
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 a_next = (ap && lkk < ld) ? *reinterpret_cast<const float4 *>(ap) : zero4;
        float4 b_next = (bp && lkk < ld) ? *reinterpret_cast<const float4 *>(bp) : zero4;
        // (every step of the tile before ended in a barrier: nobody still reads copy 0)
        *reinterpret_cast<float4 *>(&As[0][lrow][lkk]) = a_next;
        *reinterpret_cast<float4 *>(&Bs[0][lrow][lkk]) = b_next;
        __syncthreads();
        for (int k0 = 0, cur = 0; k0 < dim; k0 += PK, cur ^= 1) {
            {
                const int kn = k0 + PK + lkk;
                a_next = (ap && kn < ld) ? *reinterpret_cast<const float4 *>(ap + k0 + PK) : zero4;
                b_next = (bp && kn < ld) ? *reinterpret_cast<const float4 *>(bp + k0 + PK) : zero4;
            }
#pragma unroll
            for (int g = 0; g < PK; g += 4) {
                if (k0 + g >= dim) break;
                float4 a[4], b[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4 *>(&As[cur][ty * 4 + r][g]);
#pragma unroll
                for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const float4 *>(&Bs[cur][tx + 16 * c][g]);
                if (k0 + g < dim4) {  // a full group of four: element m feeds accumulator m
#pragma unroll
                    for (int r = 0; r < 4; ++r)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            acc[r][c][0] = __fadd_rn(acc[r][c][0], __fmul_rn(a[r].x, b[c].x));
                            acc[r][c][1] = __fadd_rn(acc[r][c][1], __fmul_rn(a[r].y, b[c].y));
                            acc[r][c][2] = __fadd_rn(acc[r][c][2], __fmul_rn(a[r].z, b[c].z));
                            acc[r][c][3] = __fadd_rn(acc[r][c][3], __fmul_rn(a[r].w, b[c].w));
                        }
                } else {  // the last 1-3 elements all go to accumulator 0, in order
                    const int rem = dim - dim4;
#pragma unroll
                    for (int r = 0; r < 4; ++r)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            acc[r][c][0] = __fadd_rn(acc[r][c][0], __fmul_rn(a[r].x, b[c].x));
                            if (rem > 1) acc[r][c][0] = __fadd_rn(acc[r][c][0], __fmul_rn(a[r].y, b[c].y));
                            if (rem > 2) acc[r][c][0] = __fadd_rn(acc[r][c][0], __fmul_rn(a[r].z, b[c].z));
                        }
                }
            }
            // the other copy was last read one step ago, before that step's barrier
            *reinterpret_cast<float4 *>(&As[cur ^ 1][lrow][lkk]) = a_next;
            *reinterpret_cast<float4 *>(&Bs[cur ^ 1][lrow][lkk]) = b_next;
            __syncthreads();
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = i0 + ty * 4 + r;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = j0 + tx + 16 * c;
                const float s = __fadd_rn(__fadd_rn(acc[r][c][0], acc[r][c][1]), __fadd_rn(acc[r][c][2], acc[r][c][3]));
                if (i < n && j < i && s >= threshold) {
                    const int pos = atomicAdd(&count[i], 1);
                    if (pos < PMAX) near[(size_t)i * PMAX + pos] = j;
                }
            }
        }
    }
}

// One warp per row: more than 256 neighbours -> overflow, list dropped; else sort ascending.
__global__ void __launch_bounds__(256) k_prescreen_finish(int n, int *__restrict__ near, int *__restrict__ count,
                                                          unsigned char *__restrict__ overflow) {
    __shared__ int buf[8][PMAX];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int i = blockIdx.x * 8 + w; i < n; i += gridDim.x * 8) {
        const int c = count[i];
        if (c > PMAX) {
            if (lane == 0) {
                overflow[i] = 1;
                count[i] = 0;
            }
            continue;
        }
        if (lane == 0) overflow[i] = 0;
        if (c < 2) continue;
        int sz = 2;
        while (sz < c) sz <<= 1;
        for (int t = lane; t < sz; t += 32) buf[w][t] = (t < c) ? near[(size_t)i * PMAX + t] : 0x7fffffff;
        __syncwarp();
        for (int size = 2; size <= sz; size <<= 1)
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int t = lane; t < (sz >> 1); t += 32) {
                    const int pos = 2 * t - (t & (stride - 1));
                    const int x = buf[w][pos], y = buf[w][pos + stride];
                    const bool asc = (pos & size) == 0;
                    if ((x > y) == asc) {
                        buf[w][pos] = y;
                        buf[w][pos + stride] = x;
                    }
                }
                __syncwarp();
            }
        for (int t = lane; t < c; t += 32) near[(size_t)i * PMAX + t] = buf[w][t];
        __syncwarp();
    }
}

struct PreBufs {
    float *d_v = nullptr;
    int *d_near = nullptr, *d_count = nullptr;
    unsigned char *d_over = nullptr;
    ~PreBufs() {
        if (d_v) cudaFree(d_v);
        if (d_near) cudaFree(d_near);
        if (d_count) cudaFree(d_count);
        if (d_over) cudaFree(d_over);
    }
};

}  // namespace lk

using namespace lk;

extern "C" int lk_prescreen_pairs(const float *vecs, int64_t n, int dim, float threshold, int device, int32_t *near,
                                  int32_t *count, uint8_t *overflow) {
    if (n < 0 || dim < 1 || dim > LK_MAX_DIM || (n > 0 && (!vecs || !near || !count || !overflow)))
        return fail(LK_EINVAL, "lk_prescreen_pairs: bad argument");
    if (n > 0x7fffff00ll / LK_PRESCREEN_MAX) return fail(LK_ERANGE, "lk_prescreen_pairs: too many vectors");
    if (n == 0) return LK_OK;
    if (lk_device_count() <= device || device < 0)
        return fail(LK_ECUDA, "lk_prescreen_pairs: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    const int ld = (dim + 3) & ~3;
    PreBufs b;
    LK_CUDA(cudaMalloc((void **)&b.d_v, (size_t)n * ld * 4));
    LK_CUDA(cudaMalloc((void **)&b.d_near, (size_t)n * PMAX * 4));
    LK_CUDA(cudaMalloc((void **)&b.d_count, (size_t)n * 4));
    LK_CUDA(cudaMalloc((void **)&b.d_over, (size_t)n));
    LK_CUDA(cudaMemset(b.d_v, 0, (size_t)n * ld * 4));
    LK_CUDA(cudaMemcpy2D(b.d_v, (size_t)ld * 4, vecs, (size_t)dim * 4, (size_t)dim * 4, (size_t)n, cudaMemcpyHostToDevice));
    LK_CUDA(cudaMemset(b.d_count, 0, (size_t)n * 4));
    const long long nt = (n + PT - 1) / PT;
    const long long tiles = nt * (nt + 1) / 2;
    int sms = 0;
    LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int grid = (int)std::min<long long>(tiles, (long long)sms * 4);
    k_prescreen_pairs<<<grid, PTHREADS>>>(b.d_v, (int)n, dim, ld, threshold, tiles, b.d_near, b.d_count);
    LK_CUDA(cudaGetLastError());
    k_prescreen_finish<<<(int)std::min<long long>((n + 7) / 8, (long long)sms * 8), 256>>>((int)n, b.d_near, b.d_count, b.d_over);
    LK_CUDA(cudaGetLastError());
    LK_CUDA(cudaMemcpy(near, b.d_near, (size_t)n * PMAX * 4, cudaMemcpyDeviceToHost));
    LK_CUDA(cudaMemcpy(count, b.d_count, (size_t)n * 4, cudaMemcpyDeviceToHost));
    LK_CUDA(cudaMemcpy(overflow, b.d_over, (size_t)n, cudaMemcpyDeviceToHost));
    return LK_OK;
}
