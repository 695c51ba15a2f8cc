// Candidate x seed scoring of face clustering: for every unassigned face the seeds whose
// float32 dot with it reaches a floor, as ascending lists with the scores.
//
// Device replacement for the arithmetic of scoreAgainstSeeds
// (media-server/tasks/face_cluster.go:1315-1462): the reference scores candidates four at a
// time against every seed (dot4, :939-967) and the last one to three candidates of a
// worker's chunk one at a time (dotf, :908-925), drops every score below
// threshold - corroborationSlack (:1417) and feeds the rest, in seed order, to its decision
// logic.  That logic (vetoes, cannot-links, corroboration counts, the mean guard) is
// sparse bookkeeping over maps and stays with the caller; this file produces exactly the
// (seed, score) pairs it consumes.
//
// Arithmetic is the reference's, bit for bit: float32 multiply and add, never fused.
//   grouped candidates   two accumulators per pair: even elements into s, odd into t, in
//                        ascending order, result s + t (an odd length's last element goes to s;
//                        rows are zero-padded to an even length, which adds exact zeros to t)
//   chunk-tail candidates four accumulators fed by element index mod 4, leftovers to the
//                        first, result (s0 + s1) + (s2 + s3)
// Which candidates are grouped depends on how the reference splits its input over workers:
// the caller passes that chunk length (0 = one chunk), so any worker count can be matched.
//
// Bound: float32 ALU (one multiply + one add per element pair); candidates and seeds
// (tens of MB) stay in L2.
#include <algorithm>
#include <string>
#include <vector>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"

namespace lk {

constexpr int ST = 64;        // tile edge: 16 groups of 4 candidates x 64 seeds
constexpr int SK = 16;        // elements of every vector staged per step
constexpr int STHREADS = 256;

struct SeedHit {
    unsigned long long key;  // candidate << 32 | seed
    float score;
    int pad;
};

// Grouped candidates.  group_base[g] = index of the first of 4 consecutive candidates.
__global__ void __launch_bounds__(STHREADS) k_seed_scores_grouped(const float *__restrict__ cands,
                                                                  const int *__restrict__ group_base, int n_groups,
                                                                  const float *__restrict__ seeds, int n_seeds, int ld,
                                                                  float min_score, SeedHit *__restrict__ hits,
                                                                  unsigned long long cap,
                                                                  unsigned long long *__restrict__ n_hits) {
    // +4: rows lie 80 B = 5 x 16 B apart.  A thread's four columns are rows tx, tx+16, tx+32, tx+48 of Bs,
    // so the eight lanes of a quarter warp read eight neighbouring rows, which fall on eight different
    // 16-byte bank groups (four neighbouring rows per thread would put them on two).
    // Two copies of each tile: while the threads compute on one, the next step's floats go into the other,
    // which leaves one barrier per step.
    __shared__ float As[2][ST][SK + 4], Bs[2][ST][SK + 4];
    __shared__ int s_base[ST / 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int g_tiles = (n_groups + ST / 4 - 1) / (ST / 4), s_tiles = (n_seeds + ST - 1) / ST;
    for (long long t = blockIdx.x; t < (long long)g_tiles * s_tiles; t += gridDim.x) {
        const int gt = (int)(t / s_tiles), st = (int)(t % s_tiles);
        const int g0 = gt * (ST / 4), j0 = st * ST;
        __syncthreads();
        if (tid < ST / 4) s_base[tid] = (g0 + tid < n_groups) ? group_base[g0 + tid] : -1;
        __syncthreads();
        float s[4][4], tt[4][4];  // [candidate of the group][seed]: even- and odd-element sums
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[r][c] = tt[r][c] = 0.0f;
        // this thread's 4 floats of the staging step: fetched one step ahead, so the L2 latency
        // hides behind the arithmetic of the step before
        const int lrow = tid >> 2, lkk = (tid & 3) * 4;
        const int lbase = s_base[lrow >> 2];
        const float *ap = (lbase >= 0) ? cands + (size_t)(lbase + (lrow & 3)) * ld + lkk : nullptr;
        const float *bp = (j0 + lrow < n_seeds) ? seeds + (size_t)(j0 + lrow) * ld + lkk : nullptr;
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 a_next = (ap && lkk < ld) ? *reinterpret_cast<const float4 *>(ap) : zero4;
        float4 b_next = (bp && lkk < ld) ? *reinterpret_cast<const float4 *>(bp) : zero4;
        // (every step of the tile before ended in a barrier: nobody still reads copy 0)
        *reinterpret_cast<float4 *>(&As[0][lrow][lkk]) = a_next;
        *reinterpret_cast<float4 *>(&Bs[0][lrow][lkk]) = b_next;
        __syncthreads();
        for (int k0 = 0, cur = 0; k0 < ld; k0 += SK, cur ^= 1) {
            {
                const int kn = k0 + SK + lkk;
                a_next = (ap && kn < ld) ? *reinterpret_cast<const float4 *>(ap + k0 + SK) : zero4;
                b_next = (bp && kn < ld) ? *reinterpret_cast<const float4 *>(bp + k0 + SK) : zero4;
            }
#pragma unroll
            for (int g = 0; g < SK; g += 4) {
                if (k0 + g >= ld) break;
                float4 a[4], b[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4 *>(&As[cur][ty * 4 + r][g]);
#pragma unroll
                for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const float4 *>(&Bs[cur][tx + 16 * c][g]);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        s[r][c] = __fadd_rn(s[r][c], __fmul_rn(a[r].x, b[c].x));
                        tt[r][c] = __fadd_rn(tt[r][c], __fmul_rn(a[r].y, b[c].y));
                        s[r][c] = __fadd_rn(s[r][c], __fmul_rn(a[r].z, b[c].z));
                        tt[r][c] = __fadd_rn(tt[r][c], __fmul_rn(a[r].w, b[c].w));
                    }
            }
            // the other copy was last read one step ago, before that step's barrier
            *reinterpret_cast<float4 *>(&As[cur ^ 1][lrow][lkk]) = a_next;
            *reinterpret_cast<float4 *>(&Bs[cur ^ 1][lrow][lkk]) = b_next;
            __syncthreads();
        }
        const int base = s_base[ty];
        if (base < 0) continue;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = j0 + tx + 16 * c;
                const float sc = __fadd_rn(s[r][c], tt[r][c]);
                if (j < n_seeds && sc >= min_score) {
                    const unsigned long long pos = atomicAdd(n_hits, 1ull);
                    if (pos < cap) {
                        hits[pos].key = ((unsigned long long)(unsigned)(base + r) << 32) | (unsigned)j;
                        hits[pos].score = sc;
                    }
                }
            }
    }
}

// Chunk-tail candidates, one (candidate, seed) pair per thread, the one-at-a-time order.
__global__ void __launch_bounds__(256) k_seed_scores_single(const float *__restrict__ cands, const int *__restrict__ tail,
                                                            int n_tail, const float *__restrict__ seeds, int n_seeds,
                                                            int dim, int ld, float min_score,
                                                            SeedHit *__restrict__ hits, unsigned long long cap,
                                                            unsigned long long *__restrict__ n_hits) {
    const long long total = (long long)n_tail * n_seeds;
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += (long long)gridDim.x * blockDim.x) {
        const int ti = (int)(p / n_seeds), j = (int)(p % n_seeds);
        const int cand = tail[ti];
        const float *a = cands + (size_t)cand * ld, *b = seeds + (size_t)j * ld;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int i = 0;
        for (; i + 4 <= dim; i += 4) {
            const float4 x = *reinterpret_cast<const float4 *>(a + i), y = *reinterpret_cast<const float4 *>(b + i);
            s0 = __fadd_rn(s0, __fmul_rn(x.x, y.x));
            s1 = __fadd_rn(s1, __fmul_rn(x.y, y.y));
            s2 = __fadd_rn(s2, __fmul_rn(x.z, y.z));
            s3 = __fadd_rn(s3, __fmul_rn(x.w, y.w));
        }
        for (; i < dim; ++i) s0 = __fadd_rn(s0, __fmul_rn(a[i], b[i]));
        const float sc = __fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2, s3));
        if (sc >= min_score) {
            const unsigned long long pos = atomicAdd(n_hits, 1ull);
            if (pos < cap) {
                hits[pos].key = ((unsigned long long)(unsigned)cand << 32) | (unsigned)j;
                hits[pos].score = sc;
            }
        }
    }
}

struct SeedBufs {
    float *d_c = nullptr, *d_s = nullptr;
    int *d_groups = nullptr, *d_tail = nullptr;
    SeedHit *d_hits = nullptr;
    unsigned long long *d_count = nullptr;
    ~SeedBufs() {
        if (d_c) cudaFree(d_c);
        if (d_s) cudaFree(d_s);
        if (d_groups) cudaFree(d_groups);
        if (d_tail) cudaFree(d_tail);
        if (d_hits) cudaFree(d_hits);
        if (d_count) cudaFree(d_count);
    }
};

}  // namespace lk

using namespace lk;

extern "C" int lk_seed_scores(const float *cands, int64_t n_cand, const float *seeds, int64_t n_seeds, int dim,
                              float min_score, int64_t chunk, int device, int64_t *row_start, int32_t *out_seed,
                              float *out_score, int64_t cap, int64_t *out_total) {
    if (n_cand < 0 || n_seeds < 0 || dim < 1 || dim > LK_MAX_DIM || chunk < 0 || cap < 0 || !row_start || !out_total ||
        (n_cand > 0 && !cands) || (n_seeds > 0 && !seeds) || (cap > 0 && (!out_seed || !out_score)))
        return fail(LK_EINVAL, "lk_seed_scores: bad argument");
    if (n_cand > 0x7fffffffll || n_seeds > 0x7fffffffll) return fail(LK_ERANGE, "lk_seed_scores: too many vectors");
    *out_total = 0;
    for (int64_t i = 0; i <= n_cand; ++i) row_start[i] = 0;
    if (n_cand == 0 || n_seeds == 0) return LK_OK;
    if (lk_device_count() <= device || device < 0)
        return fail(LK_ECUDA, "lk_seed_scores: no such CUDA device (this library has no CPU path)");
    LK_CUDA(cudaSetDevice(device));
    // Which candidates the reference scores four at a time: inside every worker chunk, groups
    // of 4 from the chunk's first candidate; what is left at the chunk's end goes one at a time
    // (media-server/tasks/face_cluster.go:1349-1360, :1375-1400).
    const int64_t ch = chunk > 0 ? chunk : n_cand;
    std::vector<int> groups, tail;
    for (int64_t lo = 0; lo < n_cand; lo += ch) {
        const int64_t hi = std::min(n_cand, lo + ch);
        int64_t b = lo;
        for (; b + 4 <= hi; b += 4) groups.push_back((int)b);
        for (; b < hi; ++b) tail.push_back((int)b);
    }
    const int ld = (dim + 3) & ~3;
    SeedBufs B;
    LK_CUDA(cudaMalloc((void **)&B.d_c, (size_t)n_cand * ld * 4));
    LK_CUDA(cudaMalloc((void **)&B.d_s, (size_t)n_seeds * ld * 4));
    LK_CUDA(cudaMemset(B.d_c, 0, (size_t)n_cand * ld * 4));
    LK_CUDA(cudaMemset(B.d_s, 0, (size_t)n_seeds * ld * 4));
    LK_CUDA(cudaMemcpy2D(B.d_c, (size_t)ld * 4, cands, (size_t)dim * 4, (size_t)dim * 4, (size_t)n_cand, cudaMemcpyHostToDevice));
    LK_CUDA(cudaMemcpy2D(B.d_s, (size_t)ld * 4, seeds, (size_t)dim * 4, (size_t)dim * 4, (size_t)n_seeds, cudaMemcpyHostToDevice));
    LK_CUDA(cudaMalloc((void **)&B.d_hits, std::max<size_t>((size_t)cap, 1) * sizeof(SeedHit)));
    LK_CUDA(cudaMalloc((void **)&B.d_count, 8));
    LK_CUDA(cudaMemset(B.d_count, 0, 8));
    int sms = 0;
    LK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    if (!groups.empty()) {
        LK_CUDA(cudaMalloc((void **)&B.d_groups, groups.size() * 4));
        LK_CUDA(cudaMemcpy(B.d_groups, groups.data(), groups.size() * 4, cudaMemcpyHostToDevice));
        const long long tiles = (long long)((groups.size() + ST / 4 - 1) / (ST / 4)) * ((n_seeds + ST - 1) / ST);
        const int grid = (int)std::min<long long>(tiles, (long long)sms * 4);
        k_seed_scores_grouped<<<grid, STHREADS>>>(B.d_c, B.d_groups, (int)groups.size(), B.d_s, (int)n_seeds, ld, min_score,
                                                  B.d_hits, (unsigned long long)cap, B.d_count);
        LK_CUDA(cudaGetLastError());
    }
    if (!tail.empty()) {
        LK_CUDA(cudaMalloc((void **)&B.d_tail, tail.size() * 4));
        LK_CUDA(cudaMemcpy(B.d_tail, tail.data(), tail.size() * 4, cudaMemcpyHostToDevice));
        const long long pairs = (long long)tail.size() * n_seeds;
        const int grid = (int)std::min<long long>((pairs + 255) / 256, (long long)sms * 8);
        k_seed_scores_single<<<grid, 256>>>(B.d_c, B.d_tail, (int)tail.size(), B.d_s, (int)n_seeds, dim, ld, min_score,
                                            B.d_hits, (unsigned long long)cap, B.d_count);
        LK_CUDA(cudaGetLastError());
    }
    unsigned long long total = 0;
    LK_CUDA(cudaMemcpy(&total, B.d_count, 8, cudaMemcpyDeviceToHost));
    *out_total = (int64_t)total;
    if ((int64_t)total > cap)
        return fail(LK_ERANGE, "lk_seed_scores: " + std::to_string(total) + " pairs reach the floor, the output holds " +
                                   std::to_string(cap) + " (the count is returned: call again with room for it)");
    std::vector<SeedHit> h((size_t)total);
    if (total) LK_CUDA(cudaMemcpy(h.data(), B.d_hits, (size_t)total * sizeof(SeedHit), cudaMemcpyDeviceToHost));
    std::sort(h.begin(), h.end(), [](const SeedHit &x, const SeedHit &y) { return x.key < y.key; });
    for (size_t i = 0; i < h.size(); ++i) {
        out_seed[i] = (int32_t)(h[i].key & 0xffffffffull);
        out_score[i] = h[i].score;
        row_start[(h[i].key >> 32) + 1]++;
    }
    for (int64_t i = 0; i < n_cand; ++i) row_start[i + 1] += row_start[i];
    return LK_OK;
}
