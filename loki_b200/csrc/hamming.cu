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
#include <string>
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

// ---------------------------------------------------------------------------
// Multi-index search (exact).  Split the 64 bits into P > radius parts: two hashes within
// `radius` bits differ in at most `radius` parts, so they agree exactly on at least one.
// For every part the hashes are bucketed by that part's value (counting sort) and only
// pairs inside a bucket are tested: for 2,000,000 hashes and radius 6 (7 parts of 9-10
// bits) that is 2.7e10 pair tests instead of 2.0e12.  A pair is reported by the FIRST
// part on which it agrees, so every pair comes out exactly once.
// ---------------------------------------------------------------------------
constexpr int kMiTile = 256;      // hashes per tile edge inside a bucket
constexpr int kMiMaxBins = 1 << 16;

struct MiParts {
    int parts;
    int off[32], width[32];
};

__device__ __forceinline__ unsigned mi_key(unsigned long long h, int off, int width) {
    return (unsigned)((h >> off) & ((1ull << width) - 1ull));
}

__global__ void k_mi_hist(const unsigned long long *__restrict__ h, long long n, int off, int width, unsigned *hist) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        atomicAdd(&hist[mi_key(h[i], off, width)], 1u);
}

// One CTA: bucket offsets (exclusive prefix of the histogram), write cursors, and the
// exclusive prefix of each bucket's number of triangular tiles.
__global__ void __launch_bounds__(1024) k_mi_scan(const unsigned *hist, int bins, unsigned *offset, unsigned *cursor,
                                                  unsigned long long *tile_prefix) {
    __shared__ unsigned long long s_cnt[1024], s_tiles[1024];
    const int tid = threadIdx.x;
    const int per = (bins + 1023) / 1024;
    unsigned long long c = 0, t = 0;
    for (int i = 0; i < per; ++i) {
        const int b = tid * per + i;
        if (b < bins) {
            const unsigned long long sz = hist[b];
            const unsigned long long nt = (sz + kMiTile - 1) / kMiTile;
            c += sz;
            t += nt * (nt + 1) / 2;
        }
    }
    s_cnt[tid] = c;
    s_tiles[tid] = t;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {  // inclusive scan
        unsigned long long a = 0, b2 = 0;
        if (tid >= d) { a = s_cnt[tid - d]; b2 = s_tiles[tid - d]; }
        __syncthreads();
        s_cnt[tid] += a;
        s_tiles[tid] += b2;
        __syncthreads();
    }
    unsigned long long co = s_cnt[tid] - c, to = s_tiles[tid] - t;
    for (int i = 0; i < per; ++i) {
        const int b = tid * per + i;
        if (b < bins) {
            offset[b] = (unsigned)co;
            cursor[b] = (unsigned)co;
            tile_prefix[b] = to;
            const unsigned long long sz = hist[b];
            const unsigned long long nt = (sz + kMiTile - 1) / kMiTile;
            co += sz;
            to += nt * (nt + 1) / 2;
        }
    }
    if (tid == 1023) {
        offset[bins] = (unsigned)s_cnt[1023];
        tile_prefix[bins] = s_tiles[1023];
    }
}

__global__ void k_mi_scatter(const unsigned long long *__restrict__ h, long long n, int off, int width, unsigned *cursor,
                             unsigned long long *sorted, unsigned *sorted_idx) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long v = h[i];
        const unsigned pos = atomicAdd(&cursor[mi_key(v, off, width)], 1u);
        sorted[pos] = v;
        sorted_idx[pos] = (unsigned)i;
    }
}

// All pairs inside every bucket of part p, tile by tile; a pair within the radius is
// emitted unless it already agreed on an earlier part.
__global__ void __launch_bounds__(kMiTile) k_mi_pairs(const unsigned long long *__restrict__ sorted,
                                                      const unsigned *__restrict__ sorted_idx,
                                                      const unsigned *__restrict__ offset,
                                                      const unsigned long long *__restrict__ tile_prefix, int bins,
                                                      MiParts mp, int p, int radius, unsigned long long tile_lo,
                                                      unsigned long long tile_hi, unsigned long long *out,
                                                      unsigned long long *count, long long cap) {
    __shared__ unsigned long long cols[kMiTile];
    __shared__ unsigned cidx[kMiTile];
    for (unsigned long long t = tile_lo + blockIdx.x; t < tile_hi; t += gridDim.x) {
        // bucket of this tile: last b with tile_prefix[b] <= t
        int lo = 0, hi = bins;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tile_prefix[mid] <= t) lo = mid; else hi = mid;
        }
        const unsigned b0 = offset[lo], sz = offset[lo + 1] - b0;
        const unsigned long long local = t - tile_prefix[lo];
        // (ti, tj), tj <= ti, from the linear index over the lower triangle
        int ti = (int)((sqrt(8.0 * (double)local + 1.0) - 1.0) * 0.5);
        while ((unsigned long long)ti * (ti + 1) / 2 > local) --ti;
        while ((unsigned long long)(ti + 1) * (ti + 2) / 2 <= local) ++ti;
        const int tj = (int)(local - (unsigned long long)ti * (ti + 1) / 2);
        const unsigned r = ti * kMiTile + threadIdx.x, c0 = tj * kMiTile;
        __syncthreads();
        {
            const unsigned c = c0 + threadIdx.x;
            cols[threadIdx.x] = (c < sz) ? sorted[b0 + c] : 0ull;
            cidx[threadIdx.x] = (c < sz) ? sorted_idx[b0 + c] : 0u;
        }
        __syncthreads();
        if (r >= sz) continue;  // no barrier below this point in the iteration
        const unsigned long long hv = sorted[b0 + r];
        const unsigned hi_idx = sorted_idx[b0 + r];
        const int ncols = (int)min((unsigned)kMiTile, sz - c0);
        const int cend = (ti == tj) ? min(ncols, (int)threadIdx.x) : ncols;  // diagonal tile: columns before the row
        for (int c = 0; c < cend; ++c) {
            const unsigned long long x = hv ^ cols[c];
            if (__popcll(x) > radius) continue;
            bool earlier = false;
            for (int q = 0; q < p; ++q) earlier |= mi_key(x, mp.off[q], mp.width[q]) == 0u;
            if (earlier) continue;
            const unsigned a = hi_idx, bb = cidx[c];
            ham_emit(out, count, cap, a < bb ? a : bb, a < bb ? bb : a);
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
    int sms = 0;
    LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    // Plan: P parts of the 64 bits (P > radius, at most 16 bits each).  Use the index when it
    // tests clearly fewer pairs than the plain sweep; otherwise (large radius, few hashes) sweep.
    MiParts mp;
    mp.parts = std::max(radius + 1, 4);
    double indexed = 0.0;
    bool use_index = mp.parts <= 16 && n >= 4096;
    if (use_index) {
        int o = 0;
        for (int p = 0; p < mp.parts; ++p) {
            mp.width[p] = 64 / mp.parts + (p < 64 % mp.parts ? 1 : 0);
            mp.off[p] = o;
            o += mp.width[p];
            indexed += (double)n * (double)n / 2.0 / (double)(1ull << mp.width[p]);
        }
        use_index = indexed * 4.0 < (double)n * (double)n / 2.0;
    }
    if (use_index) {
        unsigned long long *d_sorted = nullptr, *d_tprefix = nullptr;
        unsigned *d_sidx = nullptr, *d_hist = nullptr, *d_offset = nullptr, *d_cursor = nullptr;
        auto release = [&]() {
            if (d_sorted) cudaFree(d_sorted);
            if (d_tprefix) cudaFree(d_tprefix);
            if (d_sidx) cudaFree(d_sidx);
            if (d_hist) cudaFree(d_hist);
            if (d_offset) cudaFree(d_offset);
            if (d_cursor) cudaFree(d_cursor);
        };
        cudaError_t e = cudaMalloc((void **)&d_sorted, (size_t)n * 8);
        if (e == cudaSuccess) e = cudaMalloc((void **)&d_sidx, (size_t)n * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&d_hist, (size_t)kMiMaxBins * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&d_offset, (size_t)(kMiMaxBins + 1) * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&d_cursor, (size_t)kMiMaxBins * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&d_tprefix, (size_t)(kMiMaxBins + 1) * 8);
        for (int p = 0; p < mp.parts && e == cudaSuccess; ++p) {
            const int bins = 1 << mp.width[p];
            e = cudaMemsetAsync(d_hist, 0, (size_t)bins * 4);
            if (e != cudaSuccess) break;
            const int g = (int)std::min<long long>((n + 255) / 256, (long long)sms * 8);
            k_mi_hist<<<g, 256>>>(b.d_h, n, mp.off[p], mp.width[p], d_hist);
            k_mi_scan<<<1, 1024>>>(d_hist, bins, d_offset, d_cursor, d_tprefix);
            k_mi_scatter<<<g, 256>>>(b.d_h, n, mp.off[p], mp.width[p], d_cursor, d_sorted, d_sidx);
            unsigned long long tiles = 0;
            e = cudaMemcpy(&tiles, d_tprefix + bins, 8, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) break;
            const unsigned long long lo = tiles * (unsigned long long)part / parts;
            const unsigned long long hi = tiles * (unsigned long long)(part + 1) / parts;
            if (hi > lo) {
                const int grid = (int)std::min<unsigned long long>(hi - lo, (unsigned long long)sms * 16);
                k_mi_pairs<<<grid, kMiTile>>>(d_sorted, d_sidx, d_offset, d_tprefix, bins, mp, p, radius, lo, hi, b.d_out,
                                              b.d_count, cap);
            }
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        release();
        if (e != cudaSuccess) return fail(LK_ECUDA, std::string("lk_hamming_pairs (indexed): ") + cudaGetErrorString(e));
    } else {
        const int nt = (int)((n + kHamTile - 1) / kHamTile);
        const long long tiles = (long long)nt * (nt + 1) / 2;
        const long long lo = tiles * part / parts, hi = tiles * (part + 1) / parts;
        if (hi > lo) {
            const long long grid = std::min<long long>(hi - lo, (long long)sms * 8);
            k_hamming_pairs<<<(int)grid, kHamThreads>>>(b.d_h, n, radius, nt, lo, hi, b.d_out, b.d_count, cap);
            LK_CUDA(cudaGetLastError());
        }
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
