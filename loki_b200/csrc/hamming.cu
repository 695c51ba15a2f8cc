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
#include "comm.hpp"
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
// Stable counting sort by one digit of a 64-bit key, digit = (key >> shift) & (bins - 1),
// bins <= 4096.  It serves twice: to bucket the hashes by a bit field (below) and, as the
// pass of a least-significant-digit radix sort, to put the found pairs in order on the
// device.  Stable means: elements with equal digits keep their input order.  That makes the
// layout of every bucket a function of the input alone, which the part/parts split relies on
// (each caller re-buckets and must see the same tiles).
//
//   k_sort_count    every block tabulates its contiguous chunk: table[digit * blocks + block]
//   k_sort_scan     one CTA, exclusive prefix over the table in place (digit-major, so a
//                   digit's run starts with block 0's elements)
//   k_sort_scatter  every warp owns a contiguous piece of its block's chunk and walks it in
//                   order, 32 elements a step; equal digits inside a step are ranked by lane
// ---------------------------------------------------------------------------
constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortMaxBits = 12;
constexpr int kSortMaxBlocks = 1024;

__device__ __forceinline__ unsigned sort_digit(unsigned long long key, int shift, unsigned mask) {
    return (unsigned)(key >> shift) & mask;
}

__global__ void __launch_bounds__(kSortThreads) k_sort_count(const unsigned long long *__restrict__ keys, long long n,
                                                             long long chunk, int shift, int bins, unsigned *table) {
    extern __shared__ unsigned s_hist[];  // [bins]
    for (int b = threadIdx.x; b < bins; b += kSortThreads) s_hist[b] = 0u;
    __syncthreads();
    const long long lo = (long long)blockIdx.x * chunk, hi = min(n, lo + chunk);
    const unsigned mask = (unsigned)bins - 1u;
    for (long long i = lo + threadIdx.x; i < hi; i += kSortThreads) atomicAdd(&s_hist[sort_digit(keys[i], shift, mask)], 1u);
    __syncthreads();
    for (int b = threadIdx.x; b < bins; b += kSortThreads) table[(size_t)b * gridDim.x + blockIdx.x] = s_hist[b];
}

__global__ void __launch_bounds__(1024) k_sort_scan(unsigned *table, long long entries) {
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_carry = 0u;
    __syncthreads();
    for (long long base = 0; base < entries; base += 4096) {
        const long long i = base + (long long)tid * 4;
        unsigned v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (i + u < entries) ? table[i + u] : 0u;
        const unsigned mine = v[0] + v[1] + v[2] + v[3];
        unsigned inc = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned t = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += t;
        }
        if (lane == 31) s_warp[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            unsigned w = s_warp[lane], winc = w;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const unsigned t = __shfl_up_sync(0xffffffffu, winc, d);
                if (lane >= d) winc += t;
            }
            s_warp[lane] = winc - w;  // exclusive over warps
        }
        __syncthreads();
        unsigned run = s_carry + s_warp[warp] + inc - mine;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i + u < entries) table[i + u] = run;
            run += v[u];
        }
        __syncthreads();
        if (tid == 1023) s_carry = run;
        __syncthreads();
    }
}

// out_keys[pos] = key; out_src[pos] = the element's input position (when asked for).
template <bool kWithSrc>
__global__ void __launch_bounds__(kSortThreads) k_sort_scatter(const unsigned long long *__restrict__ keys, long long n,
                                                               long long chunk, int shift, int bins,
                                                               const unsigned *__restrict__ table,
                                                               unsigned long long *__restrict__ out_keys,
                                                               unsigned *__restrict__ out_src) {
    extern __shared__ unsigned s_base[];  // [kSortWarps][bins]: counts, then write positions, per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned mask = (unsigned)bins - 1u;
    for (int b = threadIdx.x; b < bins * kSortWarps; b += kSortThreads) s_base[b] = 0u;
    __syncthreads();
    const long long piece = chunk / kSortWarps;  // chunk is a multiple of 32 * kSortWarps
    const long long lo = (long long)blockIdx.x * chunk + (long long)warp * piece, hi = min(n, lo + piece);
    unsigned *mine = s_base + (size_t)warp * bins;
    for (long long i = lo + lane; i < hi; i += 32) atomicAdd(&mine[sort_digit(keys[i], shift, mask)], 1u);
    __syncthreads();
    for (int b = threadIdx.x; b < bins; b += kSortThreads) {
        unsigned run = table[(size_t)b * gridDim.x + blockIdx.x];
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const unsigned c = s_base[(size_t)w * bins + b];
            s_base[(size_t)w * bins + b] = run;
            run += c;
        }
    }
    __syncthreads();
    for (long long i0 = lo; i0 < hi; i0 += 32) {
        const long long i = i0 + lane;
        const bool live = i < hi;
        const unsigned long long key = live ? keys[i] : 0ull;
        const unsigned d = live ? sort_digit(key, shift, mask) : 0xffffffffu;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        const unsigned before = __popc(peers & lanemask_lt());
        unsigned pos = 0u;
        if (live && before == 0u) {  // first lane of its digit in this step
            pos = mine[d];
            mine[d] = pos + __popc(peers);
        }
        pos = __shfl_sync(0xffffffffu, pos, __ffs(peers) - 1) + before;
        if (live) {
            out_keys[pos] = key;
            if (kWithSrc) out_src[pos] = (unsigned)i;
        }
        __syncwarp();
    }
}

struct SortPlan {
    long long chunk = 0;
    int blocks = 0;
};
static SortPlan sort_plan(long long n) {
    SortPlan p;
    const long long unit = 32 * kSortWarps * 16;  // 4096 elements
    p.chunk = std::max<long long>(unit, round_up((n + kSortMaxBlocks - 1) / kSortMaxBlocks, 32 * kSortWarps));
    p.blocks = (int)std::max<long long>(1, (n + p.chunk - 1) / p.chunk);
    return p;
}
static size_t sort_table_entries(long long n) { return (size_t)sort_plan(n).blocks << kSortMaxBits; }

// One stable pass; `table` holds at least bins * blocks words.
static cudaError_t sort_pass(const unsigned long long *keys, long long n, int shift, int bits, unsigned *table,
                             unsigned long long *out_keys, unsigned *out_src, cudaStream_t st) {
    const SortPlan p = sort_plan(n);
    const int bins = 1 << bits;
    k_sort_count<<<p.blocks, kSortThreads, (size_t)bins * 4, st>>>(keys, n, p.chunk, shift, bins, table);
    k_sort_scan<<<1, 1024, 0, st>>>(table, (long long)bins * p.blocks);
    const size_t smem = (size_t)bins * kSortWarps * 4;
    if (out_src)
        k_sort_scatter<true><<<p.blocks, kSortThreads, smem, st>>>(keys, n, p.chunk, shift, bins, table, out_keys, out_src);
    else
        k_sort_scatter<false><<<p.blocks, kSortThreads, smem, st>>>(keys, n, p.chunk, shift, bins, table, out_keys, nullptr);
    return cudaGetLastError();
}

static cudaError_t sort_allow_shared_memory() {
    const int bytes = (1 << kSortMaxBits) * kSortWarps * 4;  // 128 KB: above the default limit
    cudaError_t e = cudaFuncSetAttribute(k_sort_scatter<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_sort_scatter<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    return e;
}

static int bits_for(unsigned long long values) {  // bits needed to hold 0 .. values-1
    int b = 1;
    while (b < 32 && (1ull << b) < values) ++b;
    return b;
}

// Sorts count packed pairs (i << 32 | j, i and j below n) ascending: radix passes over the bits
// of j, then of i.  The result ends up in *sorted (one of the two buffers).
static cudaError_t sort_pairs(unsigned long long *a, unsigned long long *b, long long count, long long n, unsigned *table,
                              cudaStream_t st, unsigned long long **sorted) {
    *sorted = a;
    if (count < 2) return cudaSuccess;
    const int nb = bits_for((unsigned long long)n);
    for (int word = 0; word < 2; ++word)
        for (int done = 0; done < nb;) {
            const int bits = std::min(kSortMaxBits, nb - done);
            cudaError_t e = sort_pass(a, count, word * 32 + done, bits, table, b, nullptr, st);
            if (e != cudaSuccess) return e;
            std::swap(a, b);
            done += bits;
        }
    *sorted = a;
    return cudaSuccess;
}

// (i << 32 | j) -> the two uint32 the caller reads
__global__ void k_unpack_pairs(const unsigned long long *__restrict__ packed, long long count, uint2 *__restrict__ out) {
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += (long long)gridDim.x * blockDim.x) {
        const unsigned long long v = packed[t];
        out[t] = make_uint2((unsigned)(v >> 32), (unsigned)v);
    }
}

// ---------------------------------------------------------------------------
// Multi-index search (exact).  Take P > radius disjoint bit fields of the 64 bits: two hashes
// within `radius` bits differ in at most `radius` of the fields, so they agree exactly on at
// least one.  For every field the hashes are bucketed by the field's value (the stable sort
// above) and only pairs inside a bucket are tested: for 2,000,000 hashes and radius 6 (7 fields
// of 9 bits) that is 2.7e10 pair tests instead of 2.0e12.  A pair is reported by the FIRST field
// on which it agrees, so every pair comes out exactly once.
// ---------------------------------------------------------------------------
constexpr int kMiTile = 256;  // hashes per tile edge inside a bucket

struct MiParts {
    int parts;
    int off[32], width[32];
};

__device__ __forceinline__ unsigned mi_key(unsigned long long h, int off, int width) {
    return (unsigned)((h >> off) & ((1ull << width) - 1ull));
}

// One CTA: bucket b starts at offset[b] = table[b * blocks] (the scanned sort table); also the
// exclusive prefix of each bucket's number of triangular tiles.
__global__ void __launch_bounds__(1024) k_mi_tiles(const unsigned *__restrict__ table, int blocks, int bins, unsigned n,
                                                   unsigned *offset, unsigned long long *tile_prefix) {
    __shared__ unsigned long long s_tiles[1024];
    const int tid = threadIdx.x;
    const int per = (bins + 1023) / 1024;
    auto start = [&](int b) -> unsigned { return b < bins ? table[(size_t)b * blocks] : n; };
    unsigned long long t = 0;
    for (int i = 0; i < per; ++i) {
        const int b = tid * per + i;
        if (b < bins) {
            const unsigned long long sz = start(b + 1) - start(b);
            const unsigned long long nt = (sz + kMiTile - 1) / kMiTile;
            t += nt * (nt + 1) / 2;
        }
    }
    s_tiles[tid] = t;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {  // inclusive scan
        unsigned long long a = 0;
        if (tid >= d) a = s_tiles[tid - d];
        __syncthreads();
        s_tiles[tid] += a;
        __syncthreads();
    }
    unsigned long long to = s_tiles[tid] - t;
    for (int i = 0; i < per; ++i) {
        const int b = tid * per + i;
        if (b < bins) {
            offset[b] = start(b);
            tile_prefix[b] = to;
            const unsigned long long sz = start(b + 1) - start(b);
            const unsigned long long nt = (sz + kMiTile - 1) / kMiTile;
            to += nt * (nt + 1) / 2;
        }
    }
    if (tid == 1023) {
        offset[bins] = n;
        tile_prefix[bins] = s_tiles[1023];
    }
}

// All pairs inside every bucket of field p, tile by tile; a pair within the radius is
// emitted unless it already agreed on an earlier field.
__global__ void __launch_bounds__(kMiTile) k_mi_pairs(const unsigned long long *__restrict__ sorted,
                                                      const unsigned *__restrict__ sorted_idx,
                                                      const unsigned *__restrict__ offset,
                                                      const unsigned long long *__restrict__ tile_prefix, int bins,
                                                      MiParts mp, int p, int radius, int part, int parts,
                                                      unsigned long long *out, unsigned long long *count, long long cap) {
    __shared__ unsigned long long cols[kMiTile];
    __shared__ unsigned cidx[kMiTile];
    const unsigned long long tiles = tile_prefix[bins];
    const unsigned long long tile_lo = tiles * (unsigned long long)part / parts;
    const unsigned long long tile_hi = tiles * (unsigned long long)(part + 1) / parts;
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

// Device memory of one call: a single allocation, carved up.
struct HamWork {
    unsigned char *arena = nullptr;
    unsigned long long *d_h = nullptr, *d_out = nullptr, *d_out2 = nullptr, *d_count = nullptr;
    unsigned long long *d_sorted = nullptr, *d_tprefix = nullptr;
    unsigned *d_sidx = nullptr, *d_offset = nullptr, *d_table = nullptr;
    ~HamWork() {
        if (arena) cudaFree(arena);
    }
    // n hashes, room for `cap_out` packed pairs in each of two buffers (found list + sort partner).
    cudaError_t reserve(long long n, long long cap_out) {
        size_t off = 0;
        auto take = [&](size_t bytes) {
            const size_t at = off;
            off += (size_t)round_up((int64_t)bytes, 256);
            return at;
        };
        const size_t o_h = take((size_t)n * 8), o_out = take((size_t)cap_out * 8), o_out2 = take((size_t)cap_out * 8);
        const size_t o_count = take(8), o_sorted = take((size_t)n * 8), o_sidx = take((size_t)n * 4);
        const size_t o_offset = take(((size_t)(1 << kSortMaxBits) + 1) * 4), o_tp = take(((size_t)(1 << kSortMaxBits) + 1) * 8);
        const size_t o_table = take(std::max(sort_table_entries(n), sort_table_entries(cap_out)) * 4);
        cudaError_t e = cudaMalloc((void **)&arena, off);
        if (e != cudaSuccess) return e;
        d_h = (unsigned long long *)(arena + o_h);
        d_out = (unsigned long long *)(arena + o_out);
        d_out2 = (unsigned long long *)(arena + o_out2);
        d_count = (unsigned long long *)(arena + o_count);
        d_sorted = (unsigned long long *)(arena + o_sorted);
        d_sidx = (unsigned *)(arena + o_sidx);
        d_offset = (unsigned *)(arena + o_offset);
        d_tprefix = (unsigned long long *)(arena + o_tp);
        d_table = (unsigned *)(arena + o_table);
        return cudaSuccess;
    }
};

// Enqueues this caller's share (part of parts) of the all-pairs search on `st`: the pairs found go
// to w.d_out (unordered, at most cap), their number to *w.d_count.
static cudaError_t ham_find(HamWork &w, long long n, int radius, int part, int parts, long long cap, int sms, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(w.d_count, 0, 8, st);
    if (e != cudaSuccess) return e;
    // Plan: P disjoint fields (P > radius), each at most kSortMaxBits wide.  Use the index when it
    // tests clearly fewer pairs than the plain sweep; otherwise (large radius, few hashes) sweep.
    MiParts mp;
    mp.parts = std::max(radius + 1, 4);
    double indexed = 0.0;
    bool use_index = mp.parts <= 16 && n >= 4096;
    if (use_index) {
        int o = 0;
        for (int p = 0; p < mp.parts; ++p) {
            const int span = 64 / mp.parts + (p < 64 % mp.parts ? 1 : 0);
            mp.width[p] = std::min(span, kSortMaxBits);
            mp.off[p] = o;
            o += span;
            indexed += (double)n * (double)n / 2.0 / (double)(1ull << mp.width[p]);
        }
        use_index = indexed * 4.0 < (double)n * (double)n / 2.0;
    }
    if (use_index) {
        const SortPlan sp = sort_plan(n);
        for (int p = 0; p < mp.parts; ++p) {
            const int bins = 1 << mp.width[p];
            e = sort_pass(w.d_h, n, mp.off[p], mp.width[p], w.d_table, w.d_sorted, w.d_sidx, st);
            if (e != cudaSuccess) return e;
            k_mi_tiles<<<1, 1024, 0, st>>>(w.d_table, sp.blocks, bins, (unsigned)n, w.d_offset, w.d_tprefix);
            // an upper bound of the tiles of this field sizes the grid; the kernel reads the exact split
            const double est = (double)n * (double)n / 2.0 / (double)bins / ((double)kMiTile * kMiTile) + (double)bins;
            const int grid = (int)std::min<double>(std::max(1.0, est / parts), (double)sms * 16);
            k_mi_pairs<<<grid, kMiTile, 0, st>>>(w.d_sorted, w.d_sidx, w.d_offset, w.d_tprefix, bins, mp, p, radius, part, parts,
                                                 w.d_out, w.d_count, cap);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
        }
    } else {
        const int nt = (int)((n + kHamTile - 1) / kHamTile);
        const long long tiles = (long long)nt * (nt + 1) / 2;
        const long long lo = tiles * part / parts, hi = tiles * (part + 1) / parts;
        if (hi > lo) {
            const long long grid = std::min<long long>(hi - lo, (long long)sms * 8);
            k_hamming_pairs<<<(int)grid, kHamThreads, 0, st>>>(w.d_h, n, radius, nt, lo, hi, w.d_out, w.d_count, cap);
            e = cudaGetLastError();
        }
    }
    return e;
}

// Sorts `got` packed pairs on the device and hands them to the caller as uint32 couples.
static int ham_deliver(HamWork &w, unsigned long long *list, unsigned long long *other, long long got, long long n,
                       uint32_t *pairs, cudaStream_t st) {
    if (got <= 0) return LK_OK;
    unsigned long long *sorted = nullptr;
    LK_CUDA(sort_pairs(list, other, got, n, w.d_table, st, &sorted));
    unsigned long long *spare = sorted == list ? other : list;
    k_unpack_pairs<<<(int)std::min<long long>((got + 255) / 256, 1184), 256, 0, st>>>(sorted, got, (uint2 *)spare);
    LK_CUDA(cudaGetLastError());
    LK_CUDA(cudaMemcpyAsync(pairs, spare, (size_t)got * 8, cudaMemcpyDeviceToHost, st));
    LK_CUDA(cudaStreamSynchronize(st));
    return LK_OK;
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

namespace lk {

// The whole call.  With `gather` (world > 1) this caller searches share `part` of `parts`
// = rank of world, the ranks' lists are all-gathered (counts first, then the lists padded to the
// longest) and every rank sorts the union: the structure of the reference's tiled all-pairs
// sweep whose per-worker lists are merged in order (media-server/tasks/face_cluster.go:1189-1285),
// one level up.
int ham_pairs(const uint64_t *hashes, int64_t n, int radius, int part, int parts, int device, uint32_t *pairs, int64_t cap,
              int64_t *count, const HamAllGather *gather) {
    LK_CUDA(cudaSetDevice(device));
    LK_CUDA(sort_allow_shared_memory());
    int sms = 0;
    LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    HamWork w;
    {
        cudaError_t e = w.reserve(n, std::max<long long>(cap, 1));
        if (e != cudaSuccess) return fail(LK_ENOMEM, std::string("lk_hamming_pairs: ") + cudaGetErrorString(e));
    }
    cudaStream_t st = nullptr;  // the default stream: the call is synchronous
    LK_CUDA(cudaMemcpyAsync(w.d_h, hashes, (size_t)n * 8, cudaMemcpyHostToDevice, st));
    LK_CUDA(ham_find(w, n, radius, part, parts, cap, sms, st));
    if (!gather) {
        unsigned long long total = 0;
        LK_CUDA(cudaMemcpyAsync(&total, w.d_count, 8, cudaMemcpyDeviceToHost, st));
        LK_CUDA(cudaStreamSynchronize(st));
        LK_TRY(ham_deliver(w, w.d_out, w.d_out2, std::min<long long>((long long)total, cap), n, pairs, st));
        *count = (int64_t)total;
        return LK_OK;
    }
    const int world = parts;
    // counts of every rank (the table buffer is free between the search and the sort)
    unsigned long long *d_counts = (unsigned long long *)w.d_table;
    LK_TRY((*gather)(w.d_count, d_counts, 8, st));
    std::vector<unsigned long long> counts((size_t)world);
    LK_CUDA(cudaMemcpyAsync(counts.data(), d_counts, (size_t)world * 8, cudaMemcpyDeviceToHost, st));
    LK_CUDA(cudaStreamSynchronize(st));
    long long total = 0, kept = 0, longest = 0;
    for (int r = 0; r < world; ++r) {
        const long long got = std::min<long long>((long long)counts[r], cap);
        total += (long long)counts[r];
        kept += got;
        longest = std::max(longest, got);
    }
    *count = total;
    if (kept == 0) return LK_OK;
    // gathered lists [world][longest] | union [kept] | sort partner [kept] | sort table
    struct Arena {
        unsigned char *p = nullptr;
        ~Arena() { if (p) cudaFree(p); }
    } arena;
    const size_t b_gather = (size_t)round_up((int64_t)((size_t)world * longest * 8), 256);
    const size_t b_list = (size_t)round_up((int64_t)((size_t)kept * 8), 256);
    const size_t b_table = sort_table_entries(kept) * 4;
    {
        cudaError_t e = cudaMalloc((void **)&arena.p, b_gather + 2 * b_list + b_table);
        if (e != cudaSuccess) return fail(LK_ENOMEM, std::string("lk_hamming_pairs_sharded: ") + cudaGetErrorString(e));
    }
    unsigned long long *g = (unsigned long long *)arena.p;
    unsigned long long *all = (unsigned long long *)(arena.p + b_gather), *all2 = (unsigned long long *)(arena.p + b_gather + b_list);
    LK_TRY((*gather)(w.d_out, g, (size_t)longest * 8, st));
    long long at = 0;
    for (int r = 0; r < world; ++r) {
        const long long got = std::min<long long>((long long)counts[r], cap);
        if (got > 0) LK_CUDA(cudaMemcpyAsync(all + at, g + (size_t)r * longest, (size_t)got * 8, cudaMemcpyDeviceToDevice, st));
        at += got;
    }
    HamWork sorter;  // borrows the arena's table; owns nothing
    sorter.d_table = (unsigned *)(arena.p + b_gather + 2 * b_list);
    const long long out_n = std::min<long long>(kept, cap);
    if (out_n < kept) {
        // more pairs than the caller has room for: sort all, deliver the first cap
        unsigned long long *sorted = nullptr;
        LK_CUDA(sort_pairs(all, all2, kept, n, sorter.d_table, st, &sorted));
        unsigned long long *spare = sorted == all ? all2 : all;
        k_unpack_pairs<<<(int)std::min<long long>((out_n + 255) / 256, 1184), 256, 0, st>>>(sorted, out_n, (uint2 *)spare);
        LK_CUDA(cudaGetLastError());
        LK_CUDA(cudaMemcpyAsync(pairs, spare, (size_t)out_n * 8, cudaMemcpyDeviceToHost, st));
        LK_CUDA(cudaStreamSynchronize(st));
        return LK_OK;
    }
    return ham_deliver(sorter, all, all2, kept, n, pairs, st);
}

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
    return ham_pairs(hashes, n, radius, part, parts, device, pairs, cap, count, nullptr);
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
