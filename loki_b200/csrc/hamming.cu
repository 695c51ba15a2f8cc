// 64-bit Hamming kernels for perceptual-hash duplicate detection.
//
// The reference has no counterpart (its duplicate finder compares exact content
// hashes, media-server/tasks/dedupe.go:21-29); the nearest structural relative is
// its all-pairs thresholded sweep prescreenCandidates
// (media-server/tasks/face_cluster.go:1189-1285): every pair i<j is tested and the
// survivors are reported in ascending order.
//
// k_hamming_pairs sweeps the upper triangle in 1024 x 1024 tiles.  The hashes (8 B
// each) stay cache resident, so the kernel is bound by the integer pipes: per pair
// one XOR + one POPC on the low words rejects 99.97% of random pairs, and only the
// survivors pay for the high words.
#include <algorithm>
#include <vector>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"

namespace lk {

constexpr int kHamTile = 1024;
constexpr int kHamThreads = 256;
constexpr int kHamRows = kHamTile / kHamThreads;  // row hashes per thread

__device__ __forceinline__ void ham_emit(unsigned long long *out, unsigned long long *count, long long cap,
                                         unsigned i, unsigned j) {
    const unsigned long long pos = atomicAdd(count, 1ull);
    if ((long long)pos < cap) out[pos] = ((unsigned long long)i << 32) | j;
}

// tile (bi, bj), bi <= bj, from a linear index over the upper triangle (row-major)
__device__ __forceinline__ void tile_from_linear(long long t, int nt, int *bi, int *bj) {
    // rows 0..bi-1 hold sum_{r<bi} (nt - r) tiles
    double a = (double)nt + 0.5;
    int r = (int)(a - sqrt(a * a - 2.0 * (double)t));
    if (r < 0) r = 0;
    if (r > nt - 1) r = nt - 1;
    // fix rounding
    while (r > 0 && (long long)r * nt - (long long)r * (r - 1) / 2 > t) --r;
    while ((long long)(r + 1) * nt - (long long)(r + 1) * r / 2 <= t) ++r;
    const long long start = (long long)r * nt - (long long)r * (r - 1) / 2;
    *bi = r;
    *bj = r + (int)(t - start);
}

__global__ void __launch_bounds__(kHamThreads) k_hamming_pairs(const unsigned long long *__restrict__ h, long long n,
                                                               int radius, int nt, long long tile_lo, long long tile_hi,
                                                               unsigned long long *out, unsigned long long *count,
                                                               long long cap) {
    __shared__ unsigned long long cols[kHamTile];
    for (long long t = tile_lo + blockIdx.x; t < tile_hi; t += gridDim.x) {
        int bi, bj;
        tile_from_linear(t, nt, &bi, &bj);
        const long long r0 = (long long)bi * kHamTile, c0 = (long long)bj * kHamTile;
        __syncthreads();
        for (int i = threadIdx.x; i < kHamTile; i += kHamThreads) cols[i] = (c0 + i < n) ? h[c0 + i] : 0ull;
        __syncthreads();
        unsigned rlo[kHamRows], rhi[kHamRows];
        long long rid[kHamRows];
#pragma unroll
        for (int r = 0; r < kHamRows; ++r) {
            rid[r] = r0 + threadIdx.x + (long long)r * kHamThreads;
            const unsigned long long v = (rid[r] < n) ? h[rid[r]] : 0ull;
            rlo[r] = (unsigned)v;
            rhi[r] = (unsigned)(v >> 32);
        }
        const int ncols = (int)min((long long)kHamTile, n - c0);
        // Columns go by in chunks of 8.  The common case costs XOR + POPC + one compare that
        // ORs into a per-chunk flag (no branch per pair); only a chunk with a low-word hit is
        // looked at again, pair by pair, with the high words.
        for (int cb = 0; cb < ncols; cb += 8) {
            bool any = false;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const unsigned clo = (unsigned)cols[cb + u];  // past ncols: zero padding, filtered below
#pragma unroll
                for (int r = 0; r < kHamRows; ++r) any |= __popc(rlo[r] ^ clo) <= radius;
            }
            if (any) {
                for (int u = 0; u < 8 && cb + u < ncols; ++u) {
                    const unsigned long long cv = cols[cb + u];
                    const unsigned clo = (unsigned)cv, chi = (unsigned)(cv >> 32);
                    const long long cj = c0 + cb + u;
#pragma unroll
                    for (int r = 0; r < kHamRows; ++r) {
                        const int d = __popc(rlo[r] ^ clo) + __popc(rhi[r] ^ chi);
                        if (d <= radius && rid[r] < cj && rid[r] < n) ham_emit(out, count, cap, (unsigned)rid[r], (unsigned)cj);
                    }
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256) k_hamming_scan(const unsigned long long *__restrict__ h, long long n,
                                                      unsigned long long q, int radius, unsigned long long *out,
                                                      unsigned long long *count, long long cap) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int d = __popcll(h[i] ^ q);
        if (d <= radius) {
            const unsigned long long pos = atomicAdd(count, 1ull);
            if ((long long)pos < cap) out[pos] = ((unsigned long long)i << 32) | (unsigned)d;
        }
    }
}

struct HamBufs {
    unsigned long long *d_h = nullptr, *d_out = nullptr, *d_count = nullptr;
    ~HamBufs() {
        if (d_h) cudaFree(d_h);
        if (d_out) cudaFree(d_out);
        if (d_count) cudaFree(d_count);
    }
};

}  // namespace lk

using namespace lk;

extern "C" {

int lk_hamming_pairs(const uint64_t *hashes, int64_t n, int radius, int part, int parts, int device,
                     uint32_t *pairs, int64_t cap, int64_t *count) {
    if (n < 0 || (n > 0 && !hashes) || radius < 0 || radius > 64 || cap < 0 || (cap > 0 && !pairs) || !count ||
        parts < 1 || part < 0 || part >= parts)
        return fail(LK_EINVAL, "lk_hamming_pairs: bad argument");
    if (n > 0xffffffffll) return fail(LK_ERANGE, "lk_hamming_pairs: more than 2^32 hashes");
    *count = 0;
    if (n < 2) return LK_OK;
    if (lk_device_count() <= device) return fail(LK_ECUDA, "lk_hamming_pairs: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    HamBufs b;
    const long long dcap = std::max<long long>(cap, 1);
    LK_CUDA(cudaMalloc((void **)&b.d_h, (size_t)n * 8));
    LK_CUDA(cudaMalloc((void **)&b.d_out, (size_t)dcap * 8));
    LK_CUDA(cudaMalloc((void **)&b.d_count, 8));
    LK_CUDA(cudaMemcpy(b.d_h, hashes, (size_t)n * 8, cudaMemcpyHostToDevice));
    LK_CUDA(cudaMemset(b.d_count, 0, 8));
    const int nt = (int)((n + kHamTile - 1) / kHamTile);
    const long long tiles = (long long)nt * (nt + 1) / 2;
    const long long lo = tiles * part / parts, hi = tiles * (part + 1) / parts;
    if (hi > lo) {
        int sms = 0;
        LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        const long long grid = std::min<long long>(hi - lo, (long long)sms * 8);
        k_hamming_pairs<<<(int)grid, kHamThreads>>>(b.d_h, n, radius, nt, lo, hi, b.d_out, b.d_count, cap);
        LK_CUDA(cudaGetLastError());
    }
    unsigned long long total = 0;
    LK_CUDA(cudaMemcpy(&total, b.d_count, 8, cudaMemcpyDeviceToHost));
    const long long got = std::min<long long>((long long)total, cap);
    std::vector<unsigned long long> host((size_t)got);
    if (got > 0) LK_CUDA(cudaMemcpy(host.data(), b.d_out, (size_t)got * 8, cudaMemcpyDeviceToHost));
    std::sort(host.begin(), host.end());  // (i,j) packed as i<<32|j: numeric order = lexicographic order
    for (long long t = 0; t < got; ++t) {
        pairs[2 * t] = (uint32_t)(host[t] >> 32);
        pairs[2 * t + 1] = (uint32_t)host[t];
    }
    *count = (int64_t)total;
    return LK_OK;
}

int lk_hamming_scan(const uint64_t *hashes, int64_t n, uint64_t query, int radius, int device, uint32_t *out_ids,
                    int32_t *out_dist, int64_t cap, int64_t *count) {
    if (n < 0 || (n > 0 && !hashes) || radius < 0 || cap < 0 || (cap > 0 && (!out_ids || !out_dist)) || !count)
        return fail(LK_EINVAL, "lk_hamming_scan: bad argument");
    if (n > 0xffffffffll) return fail(LK_ERANGE, "lk_hamming_scan: more than 2^32 hashes");
    *count = 0;
    if (n == 0) return LK_OK;
    if (lk_device_count() <= device) return fail(LK_ECUDA, "lk_hamming_scan: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    HamBufs b;
    const long long dcap = std::max<long long>(cap, 1);
    LK_CUDA(cudaMalloc((void **)&b.d_h, (size_t)n * 8));
    LK_CUDA(cudaMalloc((void **)&b.d_out, (size_t)dcap * 8));
    LK_CUDA(cudaMalloc((void **)&b.d_count, 8));
    LK_CUDA(cudaMemcpy(b.d_h, hashes, (size_t)n * 8, cudaMemcpyHostToDevice));
    LK_CUDA(cudaMemset(b.d_count, 0, 8));
    int sms = 0;
    LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const long long grid = std::min<long long>((n + 255) / 256, (long long)sms * 8);
    k_hamming_scan<<<(int)grid, 256>>>(b.d_h, n, query, radius, b.d_out, b.d_count, cap);
    LK_CUDA(cudaGetLastError());
    unsigned long long total = 0;
    LK_CUDA(cudaMemcpy(&total, b.d_count, 8, cudaMemcpyDeviceToHost));
    const long long got = std::min<long long>((long long)total, cap);
    std::vector<unsigned long long> host((size_t)got);
    if (got > 0) LK_CUDA(cudaMemcpy(host.data(), b.d_out, (size_t)got * 8, cudaMemcpyDeviceToHost));
    std::sort(host.begin(), host.end());
    for (long long t = 0; t < got; ++t) {
        out_ids[t] = (uint32_t)(host[t] >> 32);
        out_dist[t] = (int32_t)(uint32_t)host[t];
    }
    *count = (int64_t)total;
    return LK_OK;
}

}  // extern "C"
