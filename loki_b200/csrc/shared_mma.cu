// Shared-concept scan on the float64 tensor-core path (mma.sync m8n8k4 f64).
//
// Device replacement for SharedQuery.Scorer (media-server/embedvec/shared.go:180-220)
// and its centered wrapper (media-server/embedindex/embedindex.go:374-393) for scans
// over whole contiguous rows.  The work is a skinny matrix product
// rows[N x dim] * terms[dim x T], T <= 32, accumulated in float64 like the reference,
// followed by a scalar epilogue per row and the fused top-k selection.
//
// Why this shape.  Per SM and clock the machine offers about 64 float64 FMAs, 16
// float32->float64 conversions, 128 B of shared-memory reads and 4 issued instructions;
// at full HBM bandwidth a row element may cost 0.17 clocks.  With scalar FMAs every
// FMA needs its operands in registers of the same lane, which means many shared-memory
// reads, a large register tile and a butterfly reduction per tile.  One m8n8k4 MMA does
// 256 FMAs (8 rows x 8 terms x 4 elements) from two operand registers per lane, the sum
// over the row never crosses lanes, and an 8 x 8 block of dots is 2 registers per lane:
//   * 8 terms cost 0.125 clocks per row element on the FMA pipe, below the HBM figure,
//     so up to 8 query-side vectors the scan is memory bound;
//   * a row element is widened once per 8 rows x 8 terms (the conversion pipe is the
//     narrow one), and the terms once per 8 rows (or not at all when they fit in shared
//     memory as float64);
//   * registers are few, so the warp count is set by shared memory alone.
//
// Data movement.  A warp owns tiles of 8 consecutive rows.  A tile is brought in as
// column slices (8 rows x `slice` bytes, one bulk asynchronous copy per row) through a
// ring of two buffers per warp, completing on an mbarrier, so that the next slice is in
// flight while the current one is multiplied.  Row pitches in shared memory are chosen
// so that the 16-byte operand reads of a quarter warp fall in distinct banks.
//
// Element order.  Lane (g = lane / 4, k = lane % 4) reads 4 consecutive floats at element
// 16 c + 4 k of row g and feeds float i to MMA step i; the term operand is read at the
// same positions, so each MMA step pairs matching elements.  The order in which a row's
// products are added differs from the reference's (as it does for every parallel sum);
// products of two float32 are exact in float64 and the dot is rounded to float32 once,
// like embedvec.Cosine (media-server/embedvec/embedvec.go:52-66).
#include <algorithm>
#include <string>

#include "bulk.cuh"
#include "lk_common.cuh"
#include "mma64.cuh"
#include "shared.cuh"
#include "topk.cuh"

namespace lk {

constexpr int kMmaRows = 8;           // rows per tile (the M of the MMA)
constexpr int kMmaGroupTiles = 4;     // tiles per epilogue group: one lane per row
constexpr int kMmaMaxBufs = 4;        // most slice buffers per warp
constexpr int kMmaOfferSlack = 512;   // most keys all warps offer between two looks at the count (16 warps x 32)
#ifndef LK_MMA_MAXW
#define LK_MMA_MAXW 16
#endif
constexpr int kMmaMaxWarps = LK_MMA_MAXW;
constexpr size_t kMmaSmemLimit = 220 * 1024;

__host__ __device__ inline int mma_cand_capacity(int k) {
    int cap = 1024;
    while (cap < k + kMmaOfferSlack + 256) cap <<= 1;
    return cap;
}
__host__ __device__ inline int mma_dot_stride(int terms) { return terms | 1; }  // odd: lanes hit distinct banks

struct MmaLayout {
    int cap;
    size_t bars, dots, params, mu, terms, bufs, total;
    long long slice_pitch, term_pitch;
};

__host__ __device__ inline MmaLayout mma_layout(int k, int warps, int nbuf, int terms, long long ld, int slice,
                                                int f64terms) {
    MmaLayout L;
    L.cap = mma_cand_capacity(k);
    size_t o = (size_t)L.cap * 8 + 16;
    L.bars = o;
    o += (size_t)warps * kMmaMaxBufs * 8;
    o = (o + 15) & ~(size_t)15;
    L.dots = o;
    o += ((size_t)warps * kMmaGroupTiles * kMmaRows * mma_dot_stride(terms) * 4 + 15) & ~(size_t)15;
    L.params = o;
    o += (sizeof(SharedParams) + 15) & ~(size_t)15;
    L.mu = o;
    o += (size_t)ld;
    L.term_pitch = f64terms ? mma_pitch(2 * ld, 16) : mma_pitch(ld, 64);
    L.terms = o;
    o += (size_t)(terms + 1) * L.term_pitch;  // one more row of zeros stands in for the terms a block of 8 lacks
    o = (o + 127) & ~(size_t)127;
    L.slice_pitch = mma_pitch(slice, 64);
    L.bufs = o;
    o += (size_t)warps * nbuf * kMmaRows * L.slice_pitch;
    L.total = o;
    return L;
}

// The scalar tail of the scorer for one row, from its T dots (each already rounded to
// float32): media-server/embedvec/shared.go:186-218.  Positive i's score is recomputed in
// the second loop rather than kept, because m is not a compile-time size.
__device__ __forceinline__ double shared_row_score(const SharedParams &P, const float *d, int m, int rank, int nneg,
                                                   float gamma, float lambda) {
    double b2 = 0.0;
    for (int j = 0; j < rank; ++j) {
        const double vb = (double)d[m + j];
        b2 += vb * vb;  // exact product
    }
    double vn2 = __dsub_rn(1.0, __dmul_rn((double)gamma, b2));
    if (vn2 < 1e-6) vn2 = 1e-6;
    const double vn = sqrt(vn2);
    auto score_of = [&](int i) {
        double sv = (double)d[i];
        for (int j = 0; j < rank; ++j)
            sv = __dsub_rn(sv, __dmul_rn(__dmul_rn((double)gamma, (double)P.qb[i * rank + j]), (double)d[m + j]));
        return sv / __dmul_rn((double)P.posnorm[i], vn);
    };
    double mean = 0.0, m2 = 0.0;
    for (int i = 0; i < m; ++i) mean = __dadd_rn(mean, __dmul_rn((double)P.posw[i], score_of(i)));
    for (int i = 0; i < m; ++i) {
        const double dd = score_of(i) - mean;
        m2 = __dadd_rn(m2, __dmul_rn(__dmul_rn((double)P.posw[i], dd), dd));
    }
    double o = __dsub_rn(mean, __dmul_rn((double)lambda, sqrt(m2)));
    for (int i = 0; i < nneg; ++i) o = __dsub_rn(o, __dmul_rn((double)P.negw[i], (double)d[m + rank + i]));
    return o;
}

template <int NT, bool F64T, bool CEN>  // NT = ceil(terms / 8) blocks of 8 terms
__global__ void __launch_bounds__(kMmaMaxWarps * 32, 1) k_scan_shared_mma(const SharedArgs a, const int slice,
                                                                          const int nbuf) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int n_threads = blockDim.x, n_warps = n_threads >> 5;
    const int m = a.params->m, rank = a.params->rank, nneg = a.params->nneg;
    const int T = m + rank + nneg;
    const int TS = mma_dot_stride(T);
    const float gamma = a.params->gamma, lambda = a.params->lambda;
    const MmaLayout L = mma_layout(a.k, n_warps, nbuf, T, a.ld, slice, F64T ? 1 : 0);
    const SharedParams &P = *reinterpret_cast<const SharedParams *>(smem + L.params);  // copied below
    CandBuf buf;
    buf.k = a.k;
    buf.cap = L.cap;
    buf.limit = buf.cap - kMmaOfferSlack;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    __shared__ int s_last, s_failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, kq = lane & 3;  // operand coordinates of this lane
    float *dots = reinterpret_cast<float *>(smem + L.dots) + (size_t)warp * kMmaGroupTiles * kMmaRows * TS;
    const unsigned smem0 = smem_u32(smem);
    const unsigned bars = smem0 + (unsigned)L.bars + warp * kMmaMaxBufs * 8;           // this warp's mbarriers
    const unsigned pitch = (unsigned)L.slice_pitch;
    const unsigned bufs = smem0 + (unsigned)L.bufs + warp * nbuf * kMmaRows * pitch;   // this warp's slice buffers
    if (tid == 0) {
        for (int i = 0; i < n_warps * kMmaMaxBufs; ++i) mbar_init(reinterpret_cast<unsigned long long *>(smem + L.bars) + i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_failed = 0;
    }
    __syncthreads();

    const int n_slices = (int)((a.ld + slice - 1) / slice);
    const unsigned last_slice_bytes = (unsigned)(a.ld - (long long)(n_slices - 1) * slice);
    const long long n_tiles = (a.n + kMmaRows - 1) / kMmaRows;
    const int last_tile_rows = (int)(a.n - (n_tiles - 1) * kMmaRows);
    const long long t_lo = n_tiles * blockIdx.x / gridDim.x, t_hi = n_tiles * (blockIdx.x + 1) / gridDim.x;
    // producer cursor: the next slice to request, its buffer, and (lanes 0-7) the source of this lane's row
    long long p_tile = t_lo + warp;
    int p_slice = 0, p_buf = 0;
    const unsigned char *p_src = a.rows + (size_t)((t_lo + warp) * kMmaRows + (lane & 7)) * a.ld;
    const long long p_tile_step = (long long)n_warps * kMmaRows * a.ld - (long long)n_slices * slice;
    auto issue_next = [&]() {  // called by the whole warp
        if (p_tile >= t_hi) return;
        const unsigned bytes = (p_slice == n_slices - 1) ? last_slice_bytes : (unsigned)slice;
        const int rows = (p_tile == n_tiles - 1) ? last_tile_rows : kMmaRows;
        if (lane == 0) mbar_expect_tx_u32(bars + p_buf * 8, bytes * (unsigned)rows);
        __syncwarp();
        if (lane < rows) bulk_load_u32(bufs + (p_buf * kMmaRows + lane) * pitch, p_src, bytes, bars + p_buf * 8);
        p_src += slice;
        if (++p_slice == n_slices) {
            p_slice = 0;
            p_tile += n_warps;
            p_src += p_tile_step;
        }
        if (++p_buf == nbuf) p_buf = 0;
    };
    for (int i = 0; i < nbuf; ++i) issue_next();

    for (int i = tid; i < buf.cap; i += n_threads) buf.keys[i] = 0ull;
    if (tid == 0) {
        buf.ctrl->count = 0;
        buf.ctrl->n_done = 0;
        buf.ctrl->thr = a.floor ? __ldcg(a.floor) : 0ull;
    }
    {   // scalars, terms (plus a row of zeros) and the mean into shared memory
        const int c16 = (int)(a.ld / 16);
        for (int i = tid; i < (int)(sizeof(SharedParams) / 4); i += n_threads)
            reinterpret_cast<int *>(smem + L.params)[i] = reinterpret_cast<const int *>(a.params)[i];
        for (int i = tid; i < (T + 1) * c16; i += n_threads) {
            const int t = i / c16, j = i % c16;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < T) f = reinterpret_cast<const float4 *>(a.terms)[(size_t)t * c16 + j];
            unsigned char *dst = smem + L.terms + (size_t)t * L.term_pitch;
            if (F64T) {
                reinterpret_cast<double2 *>(dst)[2 * j] = make_double2((double)f.x, (double)f.y);
                reinterpret_cast<double2 *>(dst)[2 * j + 1] = make_double2((double)f.z, (double)f.w);
            } else {
                reinterpret_cast<float4 *>(dst)[j] = f;
            }
        }
        if (CEN)
            for (int j = tid; j < c16; j += n_threads)
                reinterpret_cast<float4 *>(smem + L.mu)[j] = reinterpret_cast<const float4 *>(a.mu)[j];
    }
    const unsigned long long bound = a.bound ? __ldcg(a.bound) : ~0ull;
    __syncthreads();

    unsigned trow_off[NT];  // this lane's term row in each block of 8: term 8 nt + g, or the row of zeros
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) trow_off[nt] = (unsigned)(min(nt * 8 + g, T) * L.term_pitch);
    double acc[NT][2][2];  // [term block][chain][fragment]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0][0] = acc[nt][0][1] = acc[nt][1][0] = acc[nt][1][1] = 0.0;
    long long tile = t_lo + warp;  // the tile being multiplied
    int s = 0;                     // its next slice
    int c_buf = 0;                 // the buffer that slice arrives in
    unsigned c_phase = 0;          // bit i: the parity buffer i completes next
    const unsigned mu_u32 = smem0 + (unsigned)L.mu, terms_u32 = smem0 + (unsigned)L.terms;
    float inv = 1.0f, cn_next = 1.0f;
    if (CEN && tile < t_hi && tile * kMmaRows + g < a.n) cn_next = a.cnorm[tile * kMmaRows + g];
    bool counted = false, failed = false;
    int g_tiles = 0;         // finished tiles whose dots wait for the epilogue
    long long tile_row = 0;  // lane i: first row of waiting tile i
    int tile_rows = 0;       // lane i: rows of it that exist
    for (;;) {
        const bool work = tile < t_hi && !failed;
        const bool flush = !failed && s == 0 && (g_tiles == kMmaGroupTiles || (!work && g_tiles > 0));
        if (flush) {
            int seen = 0;
            if (lane == 0) seen = *(volatile int *)&buf.ctrl->count;
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen <= buf.limit) {
                const int ti = lane >> 3, r = lane & 7;  // one lane per row of the group
                const long long base = __shfl_sync(0xffffffffu, tile_row, ti);
                const int nrows = __shfl_sync(0xffffffffu, tile_rows, ti);
                bool pass = false;
                unsigned long long key = 0ull;
                if (ti < g_tiles && r < nrows) {
                    const long long row = base + r;
                    const double o = shared_row_score(P, dots + (size_t)lane * TS, m, rank, nneg, gamma, lambda);
                    float out = (float)o;
                    if (CEN && a.cnorm[row] < 1e-6f) out = 0.0f;  // a row sitting on the mean scores 0
                    key = make_key(ord_from_f32(out), (unsigned)row);
                    const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
                    pass = key > thr && key < bound;
                }
                cand_offer_warp(buf, pass, key);
                g_tiles = 0;
                __syncwarp();
                continue;
            }
        } else if (work) {
            unsigned spins = 0;
            bool ready = false;
            while (!(ready = mbar_try_wait_u32(bars + c_buf * 8, (c_phase >> c_buf) & 1u)) && ++spins < kBulkSpinLimit) {}
            if (!__all_sync(0xffffffffu, ready)) {
                failed = true;  // this warp stops; the CTA reports the failure after publishing
                if (lane == 0) s_failed = 1;
                continue;
            }
            const long long row0 = tile * kMmaRows;
            if (CEN && s == 0) {  // the norm read a tile ago; now read the next tile's
                inv = (cn_next < 1e-6f) ? 0.0f : __fdiv_rn(1.0f, cn_next);
                const long long nr = row0 + (long long)n_warps * kMmaRows + g;
                cn_next = (tile + n_warps < t_hi && nr < a.n) ? a.cnorm[nr] : 1.0f;
            }
            const unsigned off = (unsigned)s * (unsigned)slice;
            const int bytes = (s == n_slices - 1) ? (int)last_slice_bytes : slice;
            unsigned a_addr = bufs + (c_buf * kMmaRows + g) * pitch + kq * 16;
            unsigned m_addr = mu_u32 + off + kq * 16;
            unsigned t_addr = terms_u32 + (F64T ? 2u : 1u) * (off + kq * 16);
            int n_full = bytes >> 6;  // groups in which every lane has data
            for (; n_full >= 4; n_full -= 4) {
                mma_group<NT, F64T, CEN, 0>(acc, a_addr, m_addr, t_addr, trow_off, inv, true);
                mma_group<NT, F64T, CEN, 64>(acc, a_addr, m_addr, t_addr, trow_off, inv, true);
                mma_group<NT, F64T, CEN, 128>(acc, a_addr, m_addr, t_addr, trow_off, inv, true);
                mma_group<NT, F64T, CEN, 192>(acc, a_addr, m_addr, t_addr, trow_off, inv, true);
                a_addr += 256;
                m_addr += 256;
                t_addr += F64T ? 512 : 256;
            }
            for (; n_full > 0; --n_full) {
                mma_group<NT, F64T, CEN, 0>(acc, a_addr, m_addr, t_addr, trow_off, inv, true);
                a_addr += 64;
                m_addr += 64;
                t_addr += F64T ? 128 : 64;
            }
            if (bytes & 63)  // a row length that is not a multiple of 64 B
                mma_group<NT, F64T, CEN, 0>(acc, a_addr, m_addr, t_addr, trow_off, inv, kq * 16 < (bytes & 63));
            __syncwarp();   // every lane has read the buffer: request the slice that reuses it
            issue_next();
            c_phase ^= 1u << c_buf;
            if (++c_buf == nbuf) c_buf = 0;
            if (++s == n_slices) {
                // lane (g, kq) holds the dots of row g with terms 8 nt + 2 kq and + 1
                float *drow = dots + (size_t)(g_tiles * kMmaRows + g) * TS;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int t = nt * 8 + 2 * kq;
                    if (t < T) drow[t] = (float)(acc[nt][0][0] + acc[nt][1][0]);
                    if (t + 1 < T) drow[t + 1] = (float)(acc[nt][0][1] + acc[nt][1][1]);
                    acc[nt][0][0] = acc[nt][0][1] = acc[nt][1][0] = acc[nt][1][1] = 0.0;
                }
                if (lane == g_tiles) {
                    tile_row = row0;
                    tile_rows = (int)min((long long)kMmaRows, a.n - row0);
                }
                ++g_tiles;
                s = 0;
                tile += n_warps;
                __syncwarp();
            }
            continue;
        } else if (!counted) {
            if (lane == 0) atomicAdd(&buf.ctrl->n_done, 1);
            counted = true;
        }
        __syncthreads();
        const int c = buf.ctrl->count, nd = buf.ctrl->n_done;
        __syncthreads();
        if (c > buf.limit || nd == n_warps) cand_prune(buf);
        if (nd == n_warps) break;
    }

    unsigned long long *mine = a.part + (size_t)blockIdx.x * a.k;
    for (int i = tid; i < a.k; i += n_threads) mine[i] = buf.keys[i];
    if (tid == 0 && a.part_cnt != nullptr) a.part_cnt[blockIdx.x] = min(buf.ctrl->count, a.k);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        if (s_failed) atomicExch(reinterpret_cast<int *>(a.ticket + 1), 1);
        __threadfence();
        s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // The last CTA merges all lists.  Its slice buffers are idle now and hold more keys than its own
    // candidate buffer: the keys above the merge's starting threshold (between k and a few k) then fit
    // in one pass; should they not, the bisecting merge starts over.
    {
        const int spare_keys = (int)(((size_t)n_warps * nbuf * kMmaRows * pitch) / 8);
        int want = buf.cap;
        while (want < 4 * a.k && want * 2 <= spare_keys) want <<= 1;
        if (want > buf.cap) {
            buf.keys = reinterpret_cast<unsigned long long *>(smem + L.bufs);
            buf.cap = want;
            buf.limit = want - kMmaOfferSlack;
        }
    }
    if (!cand_select_flat(buf, a.part, a.part_cnt, (int)gridDim.x)) cand_select_from_lists(buf, a.part, (int)gridDim.x);
    const int cnt = buf.ctrl->count;
    for (int i = tid; i < a.k; i += n_threads) {
        const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
        a.out_keys[i] = key;
        a.out_ids[i] = key ? a.shard_base + (long long)key_slot(key) : -1;
        a.out_scores[i] = key ? f32_from_ord(key_ord(key)) : 0.0f;
        if (a.out_iscores) a.out_iscores[i] = 0;
    }
    if (tid == 0) {
        int *err = reinterpret_cast<int *>(a.ticket + 1);
        const bool bad = *(volatile int *)err != 0;
        *a.out_count = bad ? -1 : cnt;  // a warp gave up on a bulk copy: the result is not valid
        *err = 0;
        *a.ticket = 0u;
    }
}

typedef void (*mma_fn)(const SharedArgs, const int, const int);

template <int NT>
static mma_fn pick_mma_nt(bool f64terms, bool centered) {
    if (f64terms) return centered ? k_scan_shared_mma<NT, true, true> : k_scan_shared_mma<NT, true, false>;
    return centered ? k_scan_shared_mma<NT, false, true> : k_scan_shared_mma<NT, false, false>;
}
static mma_fn pick_mma(int terms, bool f64terms, bool centered) {
    const int nt = (terms + 7) / 8;
    if (nt <= 1) return pick_mma_nt<1>(f64terms, centered);
    if (nt == 2) return pick_mma_nt<2>(f64terms, centered);
    if (nt == 3) return pick_mma_nt<3>(f64terms, centered);
    return pick_mma_nt<4>(f64terms, centered);
}

struct MmaPlan {
    int warps, nbuf, slice, f64terms;
    size_t smem;
};

// As many warps as fit (the multiply loop is latency bound: 16 warps with 2 buffers measured
// 835 us where 12 with 3 took 971 and 9 with 4 took 1205, same slices), then as many buffers.
// Up to 8 terms are stored widened to float64 (their conversions would otherwise share a
// narrow pipe with the rows'); more terms stay float32 and are widened once per 8 rows.
static bool mma_plan(int terms, long long ld, int k, MmaPlan *pl) {
    if (ld < 128) return false;
#ifdef LK_MMA_SLICE
    int slice = LK_MMA_SLICE;
#else
    int slice = 512;
#endif
    if (ld < slice) slice = (int)((ld + 63) / 64 * 64);
    const int f64 = terms <= 8 ? 1 : 0;
    long long best = -1;
#if defined(LK_MMA_WARPS) && defined(LK_MMA_BUFS)  // tuning builds only
    for (int w = LK_MMA_WARPS; w <= LK_MMA_WARPS; ++w)
        for (int nb = LK_MMA_BUFS; nb <= LK_MMA_BUFS; ++nb) {
#else
    for (int w = 8; w <= kMmaMaxWarps; ++w)
        for (int nb = 2; nb <= kMmaMaxBufs; ++nb) {
#endif
            const MmaLayout L = mma_layout(k, w, nb, terms, ld, slice, f64);
            if (L.total > kMmaSmemLimit) continue;
            const long long score = (long long)w * 16 + nb;  // warps first (measured), then buffers
            if (score > best) {
                best = score;
                pl->warps = w;
                pl->nbuf = nb;
                pl->slice = slice;
                pl->f64terms = f64;
                pl->smem = L.total;
            }
        }
    if (best >= 0) return true;
    for (int w = 7; w >= 4; --w) {  // many terms of a long row: fewer warps, float32 terms
        const MmaLayout L = mma_layout(k, w, 2, terms, ld, slice, 0);
        if (L.total <= kMmaSmemLimit) {
            pl->warps = w;
            pl->nbuf = 2;
            pl->slice = slice;
            pl->f64terms = 0;
            pl->smem = L.total;
            return true;
        }
    }
    return false;
}

bool shared_mma_fits(int terms, long long ld, int k) {
    MmaPlan pl;
    return mma_plan(terms, ld, k, &pl);
}

// 0 = launched, 1 = not applicable (allow-list, or the terms do not fit), else an error status.
int shared_mma_launch(const SharedArgs &a, int terms, int grid, cudaStream_t stream) {
    MmaPlan pl;
    if (a.slots != nullptr || !mma_plan(terms, a.ld, a.k, &pl)) return 1;
    mma_fn fn = pick_mma(terms, pl.f64terms != 0, a.cnorm != nullptr);
    cudaError_t e = cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
    if (e != cudaSuccess) return fail(4, std::string("shared scan attr: ") + cudaGetErrorString(e));
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long tiles = (a.n + kMmaRows - 1) / kMmaRows;
    int g = std::min(sms, grid);  // the caller sized its per-CTA scratch for `grid` CTAs
    if (tiles < g) g = (int)std::max<long long>(tiles, 1);
    fn<<<g, pl.warps * 32, pl.smem, stream>>>(a, pl.slice, pl.nbuf);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("shared scan launch: ") + cudaGetErrorString(e));
    return 0;
}

}  // namespace lk
