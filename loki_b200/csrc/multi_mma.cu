// Batched float32 search: 8 queries per pass over the corpus on the float64 tensor-core
// path (mma.sync m8n8k4 f64), each query with its own fused top-k.
//
// The reference scores one query at a time (media-server/embedindex/embedindex.go:424-457)
// with embedvec.Cosine: float32 inputs, float64 accumulation, one rounding
// (media-server/embedvec/embedvec.go:113-122).  A single-query scan of float32 rows is bound
// by HBM, and the float64 MMA pipe needs about as long for 8 right-hand vectors as HBM needs
// to deliver the rows (0.125 vs 0.17 clocks per row element and SM), so 8 queries ride one
// pass over the corpus for little more than the price of one.  Arithmetic per score is the
// single-query kernels': exact float32 x float32 products summed in float64, rounded to
// float32 once, then the centered form (dot - cq) / cnorm in float32
// (media-server/embedindex/embedindex.go:296-304); only the order of the float64 additions
// differs, as it does between any two parallel sums.
//
// Shape: one CTA per SM, up to 16 warps.  A warp owns tiles of 8 consecutive rows, brought
// in as 512-byte column slices (one bulk asynchronous copy per row, completion on an
// mbarrier) through two buffers; the 8 prepared queries sit in shared memory widened to
// float64 (float32 when that does not fit).  After a tile's last slice lane (g, kq) holds
// the dots of row g with queries 2 kq and 2 kq + 1, finishes the two scores and offers their
// keys to the queries' candidate buffers (8 buffers per CTA, pruned together by the whole
// CTA when one runs full).  Each CTA publishes 8 ranked lists; k_merge_lists merges the
// CTAs' lists per query.  Waits on copies are bounded; a warp that gives up makes the call
// return LK_ETIMEOUT.
#include <algorithm>
#include <string>

#include "bulk.cuh"
#include "lk_common.cuh"
#include "mma64.cuh"
#include "multi.cuh"
#include "topk.cuh"

namespace lk {

constexpr int kMqRows = 8;         // rows per tile (the M of the MMA)
constexpr int kMqBufs = 2;         // slice buffers per warp
constexpr int kMqMaxWarps = 16;
constexpr int kMqSlice = 512;      // bytes of every row per slice
constexpr size_t kMqSmemLimit = 220 * 1024;

// Candidate buffer of one query: room for k survivors plus what all warps can add between
// two looks at the "a buffer is filling up" flag (16 warps x 8 rows) plus slack.
__host__ __device__ inline int mq_cand_capacity(int k) {
    int cap = 512;
    while (cap < k + 2 * kMqMaxWarps * kMqRows) cap <<= 1;
    return cap;
}

struct MqLayout {
    int cap;
    size_t ctrl, bars, terms, bufs, total;
    long long slice_pitch, term_pitch;
};

__host__ __device__ inline MqLayout mq_layout(int k, int warps, long long ld, int f64terms) {
    MqLayout L;
    L.cap = mq_cand_capacity(k);
    size_t o = (size_t)kMultiQueries * L.cap * 8;  // keys[8][cap]
    L.ctrl = o;
    o += kMultiQueries * sizeof(CandCtrl) + 16;    // per-query control words, then {n_done, filling}
    L.bars = o;
    o += (size_t)warps * kMqBufs * 8;
    o = (o + 15) & ~(size_t)15;
    L.term_pitch = f64terms ? mma_pitch(2 * ld, 16) : mma_pitch(ld, 64);
    L.terms = o;
    o += (size_t)kMultiQueries * L.term_pitch;
    o = (o + 127) & ~(size_t)127;
    L.slice_pitch = mma_pitch(kMqSlice, 64);
    L.bufs = o;
    o += (size_t)warps * kMqBufs * kMqRows * L.slice_pitch;
    L.total = o;
    return L;
}

template <bool F64T>
__global__ void __launch_bounds__(kMqMaxWarps * 32, 1) k_scan_multi_mma(const MultiArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int n_threads = blockDim.x, n_warps = n_threads >> 5;
    const MqLayout L = mq_layout(a.k, n_warps, a.ld, F64T ? 1 : 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, kq = lane & 3;  // operand coordinates of this lane
    unsigned long long *keys_all = reinterpret_cast<unsigned long long *>(smem);
    CandCtrl *ctrl = reinterpret_cast<CandCtrl *>(smem + L.ctrl);
    int *n_done = reinterpret_cast<int *>(smem + L.ctrl + kMultiQueries * sizeof(CandCtrl));
    int *filling = n_done + 1;  // some buffer has passed the mark: prune before the next tile
    const int limit = L.cap - kMqMaxWarps * kMqRows;
    auto buf_of = [&](int q) {
        CandBuf b;
        b.k = a.k;
        b.cap = L.cap;
        b.limit = limit;
        b.keys = keys_all + (size_t)q * L.cap;
        b.ctrl = ctrl + q;
        return b;
    };
    __shared__ int s_failed;

    const unsigned smem0 = smem_u32(smem);
    const unsigned bars = smem0 + (unsigned)L.bars + warp * kMqBufs * 8;
    const unsigned pitch = (unsigned)L.slice_pitch;
    const unsigned bufs = smem0 + (unsigned)L.bufs + warp * kMqBufs * kMqRows * pitch;
    if (tid == 0) {
        for (int i = 0; i < n_warps * kMqBufs; ++i) mbar_init(reinterpret_cast<unsigned long long *>(smem + L.bars) + i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_failed = 0;
        *n_done = 0;
        *filling = 0;
    }
    __syncthreads();

    const int n_slices = (int)((a.ld + kMqSlice - 1) / kMqSlice);
    const unsigned last_slice_bytes = (unsigned)(a.ld - (long long)(n_slices - 1) * kMqSlice);
    const long long n_tiles = (a.n + kMqRows - 1) / kMqRows;
    const int last_tile_rows = (int)(a.n - (n_tiles - 1) * kMqRows);
    const long long t_lo = n_tiles * blockIdx.x / gridDim.x, t_hi = n_tiles * (blockIdx.x + 1) / gridDim.x;
    // producer cursor: the next slice to request, its buffer, and (lanes 0-7) the source of this lane's row
    long long p_tile = t_lo + warp;
    int p_slice = 0, p_buf = 0;
    const unsigned char *p_src = a.rows + (size_t)((t_lo + warp) * kMqRows + (lane & 7)) * a.ld;
    const long long p_tile_step = (long long)n_warps * kMqRows * a.ld - (long long)n_slices * kMqSlice;
    auto issue_next = [&]() {  // called by the whole warp
        if (p_tile >= t_hi) return;
        const unsigned bytes = (p_slice == n_slices - 1) ? last_slice_bytes : (unsigned)kMqSlice;
        const int rows = (p_tile == n_tiles - 1) ? last_tile_rows : kMqRows;
        if (lane == 0) mbar_expect_tx_u32(bars + p_buf * 8, bytes * (unsigned)rows);
        __syncwarp();
        if (lane < rows) bulk_load_u32(bufs + (p_buf * kMqRows + lane) * pitch, p_src, bytes, bars + p_buf * 8);
        p_src += kMqSlice;
        if (++p_slice == n_slices) {
            p_slice = 0;
            p_tile += n_warps;
            p_src += p_tile_step;
        }
        if (++p_buf == kMqBufs) p_buf = 0;
    };
    for (int i = 0; i < kMqBufs; ++i) issue_next();

    for (int i = tid; i < kMultiQueries * L.cap; i += n_threads) keys_all[i] = 0ull;
    if (tid < kMultiQueries) {
        ctrl[tid].count = 0;
        ctrl[tid].n_done = 0;
        ctrl[tid].thr = (tid < a.nq) ? 0ull : ~0ull;  // a query slot past the batch accepts nothing
    }
    {   // the prepared queries into shared memory, rows of the padded pitch (zeros past the batch)
        const int c16 = (int)(a.ld / 16);
        for (int i = tid; i < kMultiQueries * c16; i += n_threads) {
            const int t = i / c16, j = i % c16;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < a.nq) f = reinterpret_cast<const float4 *>(a.queries)[(size_t)t * c16 + j];
            unsigned char *dst = smem + L.terms + (size_t)t * L.term_pitch;
            if (F64T) {
                reinterpret_cast<double2 *>(dst)[2 * j] = make_double2((double)f.x, (double)f.y);
                reinterpret_cast<double2 *>(dst)[2 * j + 1] = make_double2((double)f.z, (double)f.w);
            } else {
                reinterpret_cast<float4 *>(dst)[j] = f;
            }
        }
    }
    // this lane finishes the scores of queries 2 kq and 2 kq + 1
    const float cq0 = (2 * kq < a.nq) ? a.cq[2 * kq] : 0.0f, cq1 = (2 * kq + 1 < a.nq) ? a.cq[2 * kq + 1] : 0.0f;
    __syncthreads();

    const unsigned trow_off[1] = {(unsigned)(g * L.term_pitch)};
    double acc[1][2][2];
    acc[0][0][0] = acc[0][0][1] = acc[0][1][0] = acc[0][1][1] = 0.0;
    long long tile = t_lo + warp;  // the tile being multiplied
    int s = 0;                     // its next slice
    int c_buf = 0;                 // the buffer that slice arrives in
    unsigned c_phase = 0;          // bit i: the parity buffer i completes next
    const unsigned terms_u32 = smem0 + (unsigned)L.terms;
    float cn_next = 1.0f;          // centered norm of this lane's row of the tile, read a tile ahead
    if (a.cnorm != nullptr && tile < t_hi && tile * kMqRows + g < a.n) cn_next = a.cnorm[tile * kMqRows + g];
    bool counted = false, failed = false;
    for (;;) {
        const bool work = tile < t_hi && !failed;
        int full = 0;
        if (lane == 0) full = *(volatile int *)filling;
        full = __shfl_sync(0xffffffffu, full, 0);
        if (work && (s != 0 || full == 0)) {  // a tile under way is finished first: its offers fit
            unsigned spins = 0;
            bool ready = false;
            while (!(ready = mbar_try_wait_u32(bars + c_buf * 8, (c_phase >> c_buf) & 1u)) && ++spins < kBulkSpinLimit) {}
            if (!__all_sync(0xffffffffu, ready)) {
                failed = true;  // this warp stops; the CTA reports the failure after publishing
                if (lane == 0) s_failed = 1;
                continue;
            }
            const unsigned off = (unsigned)s * (unsigned)kMqSlice;
            const int bytes = (s == n_slices - 1) ? (int)last_slice_bytes : kMqSlice;
            unsigned a_addr = bufs + (c_buf * kMqRows + g) * pitch + kq * 16;
            unsigned t_addr = terms_u32 + (F64T ? 2u : 1u) * (off + kq * 16);
            int n_full = bytes >> 6;  // groups in which every lane has data
            for (; n_full >= 4; n_full -= 4) {
                mma_group<1, F64T, false, 0>(acc, a_addr, 0u, t_addr, trow_off, 1.0f, true);
                mma_group<1, F64T, false, 64>(acc, a_addr, 0u, t_addr, trow_off, 1.0f, true);
                mma_group<1, F64T, false, 128>(acc, a_addr, 0u, t_addr, trow_off, 1.0f, true);
                mma_group<1, F64T, false, 192>(acc, a_addr, 0u, t_addr, trow_off, 1.0f, true);
                a_addr += 256;
                t_addr += F64T ? 512 : 256;
            }
            for (; n_full > 0; --n_full) {
                mma_group<1, F64T, false, 0>(acc, a_addr, 0u, t_addr, trow_off, 1.0f, true);
                a_addr += 64;
                t_addr += F64T ? 128 : 64;
            }
            if (bytes & 63)  // a row length that is not a multiple of 64 B
                mma_group<1, F64T, false, 0>(acc, a_addr, 0u, t_addr, trow_off, 1.0f, kq * 16 < (bytes & 63));
            __syncwarp();   // every lane has read the buffer: request the slice that reuses it
            issue_next();
            c_phase ^= 1u << c_buf;
            if (++c_buf == kMqBufs) c_buf = 0;
            if (++s == n_slices) {
                // lane (g, kq): row g of the tile against queries 2 kq and 2 kq + 1
                const long long row = tile * kMqRows + g;
                float s0 = (float)(acc[0][0][0] + acc[0][1][0]);  // the single rounding of embedvec.Cosine
                float s1 = (float)(acc[0][0][1] + acc[0][1][1]);
                acc[0][0][0] = acc[0][0][1] = acc[0][1][0] = acc[0][1][1] = 0.0;
                if (a.cnorm != nullptr) {
                    const float cn = cn_next;
                    s0 = (cn < 1e-6f) ? 0.0f : __fdiv_rn(__fsub_rn(s0, cq0), cn);
                    s1 = (cn < 1e-6f) ? 0.0f : __fdiv_rn(__fsub_rn(s1, cq1), cn);
                    const long long nr = row + (long long)n_warps * kMqRows;
                    cn_next = (tile + n_warps < t_hi && nr < a.n) ? a.cnorm[nr] : 1.0f;
                }
                if (row < a.n) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int q = 2 * kq + j;
                        const unsigned long long key = make_key(ord_from_f32(j ? s1 : s0), (unsigned)row);
                        if (key > *(volatile unsigned long long *)&ctrl[q].thr) {
                            const int pos = atomicAdd(&ctrl[q].count, 1);
                            keys_all[(size_t)q * L.cap + pos] = key;  // pos < cap: see the prune rule
                            if (pos >= limit) *(volatile int *)filling = 1;
                        }
                    }
                }
                s = 0;
                tile += n_warps;
                __syncwarp();
            }
            continue;
        }
        if (!work && !counted) {
            if (lane == 0) atomicAdd(n_done, 1);
            counted = true;
        }
        // Rendezvous: every warp arrives here once a buffer is filling up (or when it has no
        // rows left); all buffers above k are pruned by the whole CTA, which raises their
        // thresholds.  Between a warp's look at the flag and its arrival it finishes at most
        // one tile (8 rows per query), which is what the buffers keep free above the mark.
        __syncthreads();
        const int nd = *(volatile int *)n_done, fl = *(volatile int *)filling;
        __syncthreads();
        if (fl != 0 || nd == n_warps) {
            for (int q = 0; q < kMultiQueries; ++q) {
                const CandBuf b = buf_of(q);
                if (b.ctrl->count > a.k || nd == n_warps) cand_prune(b);
            }
            if (tid == 0) *filling = 0;
            __syncthreads();
        }
        if (nd == n_warps) break;
    }

    // ranked lists of this CTA: lists[cta][query][k]
    for (int i = tid; i < a.nq * a.k; i += n_threads) {
        const int q = i / a.k, j = i % a.k;
        a.lists[((size_t)blockIdx.x * a.nq_total + (a.q0 + q)) * a.k + j] = keys_all[(size_t)q * L.cap + j];
    }
    if (tid == 0 && s_failed && a.error != nullptr) atomicExch(a.error, 1);
}

typedef void (*mq_fn)(const MultiArgs);

struct MqPlan {
    int warps, f64terms;
    size_t smem;
};

static bool mq_plan(long long ld, int k, MqPlan *pl) {
    if (ld < 128) return false;
    for (int f64 = 1; f64 >= 0; --f64)
        for (int w = kMqMaxWarps; w >= 8; --w) {
            const MqLayout L = mq_layout(k, w, ld, f64);
            if (L.total <= kMqSmemLimit) {
                pl->warps = w;
                pl->f64terms = f64;
                pl->smem = L.total;
                return true;
            }
        }
    return false;
}

bool multi_supported(long long ld, int k) {
    MqPlan pl;
    return k >= 1 && k <= kMultiMaxK && mq_plan(ld, k, &pl);
}

int multi_grid(long long n, int sm_count) {
    const long long tiles = (n + kMqRows - 1) / kMqRows;
    return (int)std::max<long long>(1, std::min<long long>(tiles, sm_count));
}

int multi_launch(const MultiArgs &a, int grid, cudaStream_t stream) {
    MqPlan pl;
    if (!mq_plan(a.ld, a.k, &pl)) return fail(7, "batched float32 scan: rows too wide");
    mq_fn fn = pl.f64terms ? k_scan_multi_mma<true> : k_scan_multi_mma<false>;
    cudaError_t e = cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
    if (e != cudaSuccess) return fail(4, std::string("batched scan attr: ") + cudaGetErrorString(e));
    fn<<<grid, pl.warps * 32, pl.smem, stream>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("batched scan launch: ") + cudaGetErrorString(e));
    return 0;
}

}  // namespace lk
