// Batched int8 search: many queries against the corpus as an int8 x int8 -> int32
// matrix product on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators
// in tensor memory), with the top-k selection fused into the epilogue so that the
// rows x queries score matrix never exists in memory.
//
// The reference scores one query at a time (media-server/embedindex/embedindex.go:424-457);
// a batch of queries turns the same arithmetic into a dense contraction, which is the
// one place on this path where tensor cores are the right tool.  Scores are the exact
// int32 dots of the single-query scan, and ranking uses the same 64-bit keys, so the
// result is bit-identical to running the queries one by one.
//
// Two SMs share every MMA (a cluster of two CTAs, tcgen05 cta_group::2): the pair holds 256
// queries (128 per CTA, resident in shared memory) and streams corpus tiles of 256 rows, of
// which each CTA loads its own half (128 rows).  One instruction of the leader CTA multiplies
// the pair's 256 queries with the 256 rows over 32 bytes of K; each SM's tensor core produces
// its own 128 queries x 256 rows into its own tensor memory.  Against one CTA per tile this
// halves the bytes every SM pulls from L2 and the shared-memory bytes behind every MMA, which
// is what bounded the one-SM form (a resident 128-query operand plus 256 streamed rows asks
// shared memory for more bytes per clock than it has).
//
// Shape of one CTA (576 threads, one CTA per SM):
//   warp 0     TMA producer: 2-D tiled loads (128-byte swizzle, never multicast) of its half
//              of every corpus tile, [128 rows x 128 K-bytes] per stage of a ring, and of its
//              128 queries; completion is counted on the LEADER's barriers
//   warp 1     allocates tensor memory (both CTAs); in the leader it issues the MMAs
//              D[256 queries x 256 rows] += Q[256 x 32] * R[256 x 32]^T, four per 128-byte K
//              slice, and commits to the stage-free / accumulator-ready barriers of both CTAs
//   warps 2-17 epilogue: a tensor-memory lane is a query, a column a corpus row: a thread
//              reads its query's scores of 64 rows per tile, tests them against the query's
//              threshold (one register) with one add and half an OR each, and appends the few
//              survivors to its query's candidate list; two accumulator buffers (all 512
//              columns of tensor memory) let the next tile's MMAs run meanwhile.  A list that
//              fills up is cut back to its best k by a warp-wide selection (bisection on the
//              score with the keys in registers), which also raises the query's threshold;
//              lists are sorted once, at the end.
// Work is split so that every pair gets the same share and the pairs walk the corpus together (see
// gemm_split): the corpus comes from HBM about once and is served to the other query tiles by L2.
// The lists of the pairs that shared a query tile are merged by k_merge_lists.
//
// Every wait (mbarrier or otherwise) is bounded by a clock; when one runs out the CTA
// raises the error word, all roles leave their loops, tensor memory is freed and the
// host reports LK_ETIMEOUT.  No load is multicast; every GPU reads only its own memory.
#include <cuda.h>

#include <algorithm>
#include <string>

#include "../../include/lokiscan.h"
#include "gemm.cuh"
#include "lk_common.cuh"
#include "scan.cuh"

namespace lk {

constexpr int GN = 128;            // queries per CTA (tensor-memory lanes); the pair's MMA has M = 256
constexpr int GM = 256;            // corpus rows per tile (MMA N, tensor-memory columns)
constexpr int GR = GM / 2;         // corpus rows of a tile that each CTA of the pair loads
constexpr int GSLICE = 128;        // K bytes per shared-memory slice: one swizzle row
constexpr int GQ_SLICE_BYTES = GN * GSLICE;  // 16 KB: one K slice of a CTA's 128 queries
constexpr int GSLICE_BYTES = GR * GSLICE;    // 16 KB: one K slice of a CTA's half of a corpus tile
constexpr int GPARTS = 4;          // epilogue warps per 32 queries: each takes a quarter of a tile's columns
constexpr int GSUB = 256;          // keys in one thread's own candidate list (a query has GPARTS of them)
constexpr int GCAP_MAX = GPARTS * GSUB;  // candidate keys a query holds between cuts (k <= 256)
constexpr int GEPI_WARPS = 16;     // epilogue warps: four per tensor-memory lane quadrant, 32 queries each
constexpr int GEPI_THREADS = GEPI_WARPS * 32;
constexpr int GTHREADS = 64 + GEPI_THREADS;
constexpr int GACC = 2;            // accumulators in tensor memory: 2 x 256 columns = all 512
constexpr int GSORT_BYTES = 8192;  // shared-memory scratch in which the final lists are sorted
// Every epilogue thread appends to a list of its own (its query, its quarter of the columns) and
// keeps the count in a register: no atomics and no shared memory on that path.  One tile adds at
// most 64 keys to a thread's list, so a cut is called for when a list holds more than GSUB - 64 at the
// end of a tile.  A cut selects the best k of a query's four lists together and deals them back out,
// k/4 to each list.
constexpr int GSUB_LIMIT = GSUB - 64;
constexpr long long GWAIT_CLOCKS = 4000000000ll;  // ~2 s at 2 GHz

__device__ __forceinline__ unsigned g_smem(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void g_mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(g_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void g_mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(g_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void g_mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(g_smem(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when the clock ran out or
// another role of this CTA has already given up.
__device__ __forceinline__ bool g_mbar_wait(unsigned long long *bar, unsigned parity, volatile int *cta_failed) {
    {   // usually the phase is already complete: no clock read on that path
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(g_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    const long long t0 = clock64();
    for (;;) {
        // the thread sleeps inside the instruction until the phase completes or the hint (in ns) runs
        // out: a waiting role issues next to nothing and leaves shared memory to the tensor core
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(g_smem(bar)), "r"(parity), "r"(4000u)
            : "memory");
        if (ok) return true;
        if (*cta_failed != 0 || clock64() - t0 > GWAIT_CLOCKS) {
            *cta_failed = 1;
            return false;
        }
    }
}
// The whole (converged) warp waits for a phase, but only lane 0 polls the barrier: 18 warps of
// pollers would compete with the MMAs' operand reads for shared memory.
__device__ __forceinline__ bool g_mbar_wait_warp(unsigned long long *bar, unsigned parity, volatile int *cta_failed) {
    int ok = 0;
    if ((threadIdx.x & 31) == 0) ok = g_mbar_wait(bar, parity, cta_failed) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// One lane of the (converged) warp: the issuer of a single-thread instruction.
__device__ __forceinline__ bool g_elect_one() {
    unsigned pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
// Address of `local` (a shared-memory address of this CTA) as it sits in the pair's leader CTA.
__device__ __forceinline__ unsigned g_leader_addr(unsigned local) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(local));
    return r;
}
__device__ __forceinline__ unsigned g_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// One arrival on a barrier of the leader CTA (which may be this CTA).
__device__ __forceinline__ void g_mbar_arrive_leader(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(g_leader_addr(g_smem(bar))) : "memory");
}
// All threads of both CTAs of the pair.
__device__ __forceinline__ void g_pair_sync() {
    asm volatile("barrier.cluster.arrive.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
// 2-D tiled TMA load into THIS CTA's shared memory: box at (x = byte column, y = row) of the tensor
// map; the bytes are counted on a barrier of the pair's leader (`leader_bar`, from g_leader_addr).
// Not a multicast load: each CTA of the pair fetches its own half of a tile.  `keep` asks L2 to
// hold on to the lines (evict-last): a corpus tile is wanted again by the pairs of every other
// query tile within microseconds, while the candidate keys written meanwhile are not.
constexpr unsigned long long G_L2_EVICT_NORMAL = 0x1000000000000000ull, G_L2_EVICT_LAST = 0x14F0000000000000ull;
__device__ __forceinline__ void g_tma_load_2d(void *dst, const CUtensorMap *tm, int x, int y, unsigned leader_bar, bool keep) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
            g_smem(dst)),
        "l"(reinterpret_cast<unsigned long long>(tm)), "r"(x), "r"(y), "r"(leader_bar),
        "l"(keep ? G_L2_EVICT_LAST : G_L2_EVICT_NORMAL)
        : "memory");
}
// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ unsigned long long g_smem_desc(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3ffffu) >> 4);        // start address
    d |= (unsigned long long)1 << 16;                          // leading byte offset (unused with swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (unsigned long long)1 << 46;                          // descriptor version
    d |= (unsigned long long)2 << 61;                          // SWIZZLE_128B
    return d;
}
// Instruction descriptor: int8 x int8 (both signed, K-major) -> int32; over the pair M = 256 queries,
// N = 256 rows.
constexpr unsigned G_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(GM >> 3) << 17) | ((unsigned)((2 * GN) >> 4) << 24);

__device__ __forceinline__ void g_mma_i8(unsigned tmem_d, unsigned long long da, unsigned long long db, bool accumulate) {
    const unsigned acc = accumulate ? 1u : 0u, z = 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(da), "l"(db), "r"(G_IDESC), "r"(acc), "r"(z)
        : "memory");
}
// Arrive on the barrier at this address in BOTH CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void g_mma_commit(unsigned long long *bar) {
    const unsigned short both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     g_smem(bar)),
                 "h"(both)
                 : "memory");
}
__device__ __forceinline__ void g_tmem_ld32(unsigned taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// Work split over P pairs for `qtiles` tiles of 256 queries and `n_tiles` corpus tiles of 256 rows.
// Two things are wanted at once: equal work per pair, and pairs that walk the corpus together, so
// that a corpus tile fetched from HBM for one query tile is found in L2 by the pairs of all the
// others (the corpus does not fit in L2; pairs at unrelated places would each stream it from HBM).
//   * D = P / qtiles pairs are dedicated to every query tile: dedicated pair s of a query tile takes
//     the corpus tiles s, s + D, s + 2D, ... below X.  All dedicated pairs advance at the same rate.
//   * The other F = P - D * qtiles pairs ("floaters") share what is left, the tiles [X, n_tiles) of
//     every query tile, as equal contiguous runs of (query tile, corpus tile) units in query-major
//     order; X = n_tiles * D * qtiles / P makes a floater's run as long as a dedicated pair's share.
//     With more query tiles than pairs (D = 0) every pair is a floater and X = 0.
// A stretch of a pair's work inside one query tile is a segment: it has its own resident queries,
// thresholds and result list (`slice` numbers the lists of a query tile).
struct GemmSplit {
    int pairs, qtiles, D, F;
    long long n_tiles, X, tail, units;  // tail = n_tiles - X, units = qtiles * tail (the floaters' units)
};
__host__ __device__ inline GemmSplit gemm_split(int pairs, int qtiles, long long n_tiles) {
    GemmSplit sp;
    sp.pairs = pairs;
    sp.qtiles = qtiles;
    sp.n_tiles = n_tiles;
    sp.D = pairs / qtiles;
    sp.F = pairs - sp.D * qtiles;
    sp.X = sp.F == 0 ? n_tiles : n_tiles * sp.D * qtiles / pairs;
    sp.tail = n_tiles - sp.X;
    sp.units = sp.tail * qtiles;
    return sp;
}
__host__ __device__ inline long long gemm_float_lo(const GemmSplit &sp, int f) { return sp.units * f / sp.F; }
// The floater whose run holds unit u.
__host__ __device__ inline int gemm_float_owner(const GemmSplit &sp, long long u) {
    int f = (int)((u * sp.F) / sp.units);
    while (f + 1 < sp.F && gemm_float_lo(sp, f + 1) <= u) ++f;
    while (f > 0 && gemm_float_lo(sp, f) > u) --f;
    return f;
}

// One stretch of a pair's work inside one query tile: corpus tiles t0, t0 + stride, ... below t1.
struct GemmSegment {
    int qt;               // 256-query tile
    long long t0, t1;
    int stride;
    int slice;            // which of the query tile's result lists this pair writes
};
// Segment `i` of pair `pair`; false when the pair has fewer.
__host__ __device__ inline bool gemm_segment(const GemmSplit &sp, int pair, int i, GemmSegment *sg) {
    const int dedicated = sp.D * sp.qtiles;
    if (pair < dedicated) {
        if (i != 0 || sp.X == 0) return false;
        sg->qt = pair / sp.D;
        sg->slice = pair % sp.D;
        sg->t0 = sg->slice;
        sg->t1 = sp.X;
        sg->stride = sp.D;
        return sg->t0 < sg->t1;
    }
    if (sp.units == 0) return false;
    const int f = pair - dedicated;
    long long u = gemm_float_lo(sp, f);
    const long long u_end = gemm_float_lo(sp, f + 1);
    for (int j = 0; u < u_end; ++j) {
        const long long qt = u / sp.tail, o0 = u - qt * sp.tail;
        const long long o1 = o0 + (u_end - u) < sp.tail ? o0 + (u_end - u) : sp.tail;
        if (j == i) {
            sg->qt = (int)qt;
            sg->t0 = sp.X + o0;
            sg->t1 = sp.X + o1;
            sg->stride = 1;
            sg->slice = sp.D + (f - gemm_float_owner(sp, qt * sp.tail));
            return true;
        }
        u += o1 - o0;
    }
    return false;
}

struct GemmShared {  // control words behind the data regions (same offsets in both CTAs of a pair)
    unsigned long long full[8], empty[8];     // corpus stages: filled (leader's is used) / free again (both)
    unsigned long long q_full, q_empty;       // resident queries: loaded (leader's) / no longer read (both)
    unsigned long long tmem_full[GACC], tmem_empty[GACC];  // accumulators: complete (both) / drained (leader's)
    unsigned long long thr[GN];  // per query: keys must exceed this to enter its list
    alignas(16) int thr_score[GN];  // score part of thr: the cheap first test (score >= thr_score)
    int cnt4[GN][GPARTS];        // per query and column quarter: keys in that list (as of the last cut or publication)
    unsigned tmem_base;
    int failed;           // any role gave up waiting
    int epilogue_failed;  // written by epilogue threads only (their common exit decision)
};

// Sort sz (a power of two) keys in this warp's scratch, descending.
__device__ inline void g_warp_sort_desc(unsigned long long *s, int sz, int lane) {
    for (int size = 2; size <= sz; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = lane; i < (sz >> 1); i += 32) {
                const int pos = 2 * i - (i & (stride - 1));
                const unsigned long long x = s[pos], y = s[pos + stride];
                const bool desc = (pos & size) == 0;
                if ((x < y) == desc) {
                    s[pos] = y;
                    s[pos + stride] = x;
                }
            }
            __syncwarp();
        }
    }
}

// Cut query q's list (global memory, unordered) back to its best k keys and raise the query's
// threshold to the k-th.  No sort: the k-th largest key is found by bisection on the score
// word with warp-wide counts (the keys sit in registers, KPL per lane), ties on that score
// are settled by a second bisection on the slot word, and the keepers are compacted in place.
template <int KPL>
__device__ inline void g_select_query(GemmShared *ctl, unsigned long long *cand_q, int q, int k, int lane) {
    int total = 0;
#pragma unroll
    for (int p = 0; p < GPARTS; ++p) total += ctl->cnt4[q][p];
    if (total <= k) return;
    unsigned hi[KPL], lo[KPL];  // score word (0 = no key: below every real one) and slot word
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        const int i = lane + 32 * u;  // list i / GSUB, entry i % GSUB
        const bool live = (i & (GSUB - 1)) < ctl->cnt4[q][i / GSUB];
        const unsigned long long key = live ? __ldcg(cand_q + i) : 0ull;
        hi[u] = (unsigned)(key >> 32);
        lo[u] = (unsigned)key;
    }
    unsigned mx = 0, mn = 0xffffffffu;
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        mx = max(mx, hi[u]);
        if (hi[u] != 0u) mn = min(mn, hi[u]);
    }
    mx = __reduce_max_sync(0xffffffffu, mx);
    mn = __reduce_min_sync(0xffffffffu, mn);
    // X = the largest score word x with count(hi >= x) >= k;  count(hi >= mn) = total > k
    unsigned a = mn, b = mx + 1u;  // count(hi >= a) >= k, count(hi >= b) < k
    while (b - a > 1u) {
        const unsigned mid = a + ((b - a) >> 1);
        int c = 0;
#pragma unroll
        for (int u = 0; u < KPL; ++u) c += (hi[u] >= mid) ? 1 : 0;
        c = __reduce_add_sync(0xffffffffu, c);
        if (c >= k) a = mid; else b = mid;
    }
    const unsigned X = a;
    int c_gt = 0, c_eq = 0;
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        c_gt += (hi[u] > X) ? 1 : 0;
        c_eq += (hi[u] == X) ? 1 : 0;
    }
    c_gt = __reduce_add_sync(0xffffffffu, c_gt);
    c_eq = __reduce_add_sync(0xffffffffu, c_eq);
    const int need = k - c_gt;  // 1 <= need <= c_eq keys of score X stay: those with the largest slot words
    unsigned Y = 0u;
    if (need < c_eq) {  // rare: more equal scores than places
        unsigned long long ya = 0ull, yb = 0x100000000ull;  // count(tie && lo >= ya) >= need > count(tie && lo >= yb)
        while (yb - ya > 1ull) {
            const unsigned long long mid = ya + ((yb - ya) >> 1);
            int c = 0;
#pragma unroll
            for (int u = 0; u < KPL; ++u) c += (hi[u] == X && lo[u] >= mid) ? 1 : 0;
            c = __reduce_add_sync(0xffffffffu, c);
            if (c >= need) ya = mid; else yb = mid;
        }
        Y = (unsigned)ya;
    }
    // the keepers, numbered r = 0 .. k-1 in lane order, go back to list r % GPARTS, entry r / GPARTS;
    // every store comes behind all loads (the keys sit in registers)
    int mine = 0;
    unsigned ymin = 0xffffffffu;
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        const bool keep = hi[u] > X || (hi[u] == X && lo[u] >= Y);
        mine += keep ? 1 : 0;
        if (hi[u] == X && lo[u] >= Y) ymin = min(ymin, lo[u]);
    }
    int pos = mine;
#pragma unroll
    for (int w = 1; w < 32; w <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, pos, w);
        if (lane >= w) pos += o;
    }
    pos -= mine;
    ymin = __reduce_min_sync(0xffffffffu, ymin);
    __syncwarp();
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        const bool keep = hi[u] > X || (hi[u] == X && lo[u] >= Y);
        if (keep) {
            __stcg(cand_q + (pos % GPARTS) * GSUB + pos / GPARTS, ((unsigned long long)hi[u] << 32) | lo[u]);
            ++pos;
        }
    }
    __syncwarp();
    if (lane < GPARTS) ctl->cnt4[q][lane] = (k + GPARTS - 1 - lane) / GPARTS;
    if (lane == 0) {
        const unsigned long long kth = ((unsigned long long)X << 32) | ymin;  // the smallest key kept
        if (kth > ctl->thr[q]) {
            ctl->thr[q] = kth;
            ctl->thr_score[q] = i32_from_ord(X);
        }
    }
    __syncwarp();
}

// Key number r of a query's lists once they hold `total` keys dealt out by g_select_query, or in any
// case the r-th in the order list 0 entry 0, list 1 entry 0, ... (used to read the final k back).
__device__ __forceinline__ unsigned long long g_dealt_key(const unsigned long long *cand_q, int r) {
    return __ldcg(cand_q + (r % GPARTS) * GSUB + r / GPARTS);
}

__device__ inline void g_prune_query(GemmShared *ctl, unsigned long long *cand_q, int q, int k, int lane) {
    g_select_query<GCAP_MAX / 32>(ctl, cand_q, q, k, lane);
}

__global__ void __launch_bounds__(GTHREADS, 1)
k_gemm_i8_topk(const __grid_constant__ CUtensorMap tm_rows, const __grid_constant__ CUtensorMap tm_queries,
               const GemmArgs a) {
    extern __shared__ unsigned char g_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address
    unsigned char *smem = g_raw + ((1024u - (g_smem(g_raw) & 1023u)) & 1023u);
    unsigned char *sm_q = smem;                                        // [ks][128 queries][128 B]: this CTA's half of the MMA's A operand
    unsigned char *sm_r = sm_q + (size_t)a.ks * GQ_SLICE_BYTES;        // [stages][128 rows][128 B]: its half of the B operand
    unsigned long long *sm_sort = reinterpret_cast<unsigned long long *>(sm_r + (size_t)a.stages * GSLICE_BYTES);  // GSORT_BYTES
    GemmShared *ctl = reinterpret_cast<GemmShared *>(sm_r + (size_t)a.stages * GSLICE_BYTES + GSORT_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rank = (int)g_cta_rank();          // 0 = the pair's leader
    const int pair = (int)(blockIdx.x >> 1), pairs = (int)(gridDim.x >> 1);
    const long long n_tiles = (a.n + GM - 1) / GM;
    const GemmSplit sp = gemm_split(pairs, a.qtiles, n_tiles);

    if (tid == 0) {
        for (int i = 0; i < a.stages; ++i) {
            g_mbar_init(&ctl->full[i], 1);
            g_mbar_init(&ctl->empty[i], 1);
        }
        g_mbar_init(&ctl->q_full, 1);
        g_mbar_init(&ctl->q_empty, 1);
        for (int i = 0; i < GACC; ++i) {
            g_mbar_init(&ctl->tmem_full[i], 1);
            g_mbar_init(&ctl->tmem_empty[i], 2 * GEPI_WARPS);  // one arrival per epilogue warp of both CTAs
        }
        ctl->failed = 0;
        ctl->epilogue_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor memory: GACC accumulators x 256 columns, in both CTAs of the pair
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(g_smem(&ctl->tmem_base)),
                     "r"(GACC * GM)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    g_pair_sync();  // the partner's barriers exist before anything is signalled across
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = ctl->tmem_base;
    volatile int *failed = &ctl->failed;

    // The two single-thread roles run their loops with the whole warp (uniform control flow,
    // warp-uniform values: loop state and descriptors can live in uniform registers, which the
    // TMA and MMA instructions take their operands from) and let one elected lane issue.
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        const unsigned q_full_leader = g_leader_addr(g_smem(&ctl->q_full));
        int stage = 0;
        unsigned phase = 0;
        bool ok = true;
        GemmSegment sg;
        for (int i = 0; ok && gemm_segment(sp, pair, i, &sg); ++i) {
            // the queries of the previous segment are no longer read once its last MMA has completed
            if (i > 0) ok = g_mbar_wait_warp(&ctl->q_empty, (unsigned)((i - 1) & 1), failed);
            if (!ok) break;
            if (g_elect_one()) {
                if (rank == 0) g_mbar_expect_tx(&ctl->q_full, (unsigned)(2 * a.ks * GQ_SLICE_BYTES));
                for (int s = 0; s < a.ks; ++s)
                    g_tma_load_2d(sm_q + (size_t)s * GQ_SLICE_BYTES, &tm_queries, s * GSLICE, sg.qt * 2 * GN + rank * GN,
                                  q_full_leader, false);
            }
            __syncwarp();
            for (long long t = sg.t0; ok && t < sg.t1; t += sg.stride) {
                for (int s = 0; s < a.ks; ++s) {
                    ok = g_mbar_wait_warp(&ctl->empty[stage], phase ^ 1u, failed);
                    if (!ok) break;
                    if (g_elect_one()) {
                        if (rank == 0) g_mbar_expect_tx(&ctl->full[stage], (unsigned)(2 * GSLICE_BYTES));
                        g_tma_load_2d(sm_r + (size_t)stage * GSLICE_BYTES, &tm_rows, s * GSLICE, (int)(t * GM + rank * GR),
                                      g_leader_addr(g_smem(&ctl->full[stage])), true);
                    }
                    __syncwarp();
                    if (++stage == a.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------ MMA issuer (leader CTA) ------------------------------
        const unsigned long long dr0 = g_smem_desc(g_smem(sm_r)), dq0 = g_smem_desc(g_smem(sm_q));
        int stage = 0, acc = 0;
        unsigned phase = 0, acc_phase = 0;
        bool ok = true;
        GemmSegment sg;
        for (int i = 0; ok && gemm_segment(sp, pair, i, &sg); ++i) {
            ok = g_mbar_wait_warp(&ctl->q_full, (unsigned)(i & 1), failed);
            for (long long t = sg.t0; ok && t < sg.t1; t += sg.stride) {
                ok = g_mbar_wait_warp(&ctl->tmem_empty[acc], acc_phase ^ 1u, failed);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned d = tmem_base + (unsigned)(acc * GM);
                for (int s = 0; s < a.ks; ++s) {
                    ok = g_mbar_wait_warp(&ctl->full[stage], phase, failed);
                    if (!ok) break;
                    // (no tcgen05 fence here: the stage was filled by TMA, whose completion on the mbarrier
                    // orders it for the MMAs; a fence per slice drained the MMA queue at every slice)
                    // the start-address field counts 16-byte units: one slice further = + 1024
                    const unsigned long long dr = dr0 + (unsigned long long)(stage * (GSLICE_BYTES >> 4));   // corpus rows
                    const unsigned long long dq = dq0 + (unsigned long long)(s * (GQ_SLICE_BYTES >> 4));     // queries
                    if (g_elect_one()) {
#pragma unroll
                        for (int k4 = 0; k4 < GSLICE / 32; ++k4)  // 32 K-bytes per MMA: +2 in 16-byte units
                            g_mma_i8(d, dq + (unsigned long long)(2 * k4), dr + (unsigned long long)(2 * k4), (s | k4) != 0);
                        g_mma_commit(&ctl->empty[stage]);  // the stage is free (in both CTAs) once these MMAs have read it
                    }
                    __syncwarp();
                    if (++stage == a.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (g_elect_one()) g_mma_commit(&ctl->tmem_full[acc]);  // accumulator complete, in both CTAs
                __syncwarp();
                if (++acc == GACC) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            if (ok && g_elect_one()) g_mma_commit(&ctl->q_empty);  // the segment's queries may be replaced
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ------------------------------ epilogue ------------------------------
        // 16 warps.  A tensor-memory lane is a query, a column a corpus row of the tile.  A warp may
        // read the lanes 32 * (warp % 4) .. + 31 (the hardware's rule), i.e. 32 queries, and takes
        // one quarter of the 256 columns: one query x 64 corpus rows per thread and tile, so the
        // threshold is one register and every survivor of a thread goes to the thread's own query.
        // The four warps that share 32 queries (a "quad") meet at their own barrier once per tile
        // and cut their lists together; the quads run independently of each other.
        const int ew = warp - 2;       // 0..15
        const int quad = warp & 3;
        const int part = ew >> 2;      // which quarter of the columns
        const int c0 = part * 64;
        const int q = quad * 32 + lane;  // this thread's query within the CTA's 128
        const int qbar = 1 + quad;       // named barrier of this quad (128 threads)
        unsigned long long *cand = a.cand + (size_t)blockIdx.x * GN * GCAP_MAX;
        unsigned long long *my_list = cand + (size_t)q * GCAP_MAX + part * GSUB;
        int acc = 0;
        unsigned acc_phase = 0;
        bool ok = true;
        GemmSegment sg;
        for (int i = 0; ok && gemm_segment(sp, pair, i, &sg); ++i) {
            const int q0 = sg.qt * 2 * GN + rank * GN;  // first query of this CTA in this segment
            unsigned long long *gthr = a.gthr + q0;     // thresholds shared by the pairs working on these queries
            if (part == 0) {
                const bool live = q0 + q < a.nq;  // queries past the end accept nothing
                const unsigned long long t0 = live ? __ldcg(gthr + q) : ~0ull;
                ctl->thr[q] = t0;
                // every real score is far inside +-2^30
                ctl->thr_score[q] = live ? (t0 ? i32_from_ord(key_ord(t0)) : -(1 << 30)) : (1 << 30);
            }
            asm volatile("bar.sync %0, 128;" ::"r"(qbar) : "memory");
            // this thread's filter and list state live in registers between the quad's meetings
            int ts = ctl->thr_score[q];
            unsigned long long thr = ctl->thr[q];
            int cnt = 0;
            int step = 0;
            for (long long t = sg.t0; t < sg.t1; t += sg.stride, ++step) {
                const bool have = g_mbar_wait_warp(&ctl->tmem_full[acc], acc_phase, failed);
                if (!have) ctl->epilogue_failed = 1;  // read by all epilogue threads behind the barrier below
                if (have) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const long long row0 = t * GM + c0;
                    const int rows_here = (int)min((long long)64, a.n - row0);  // columns past the corpus hold zeros
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        int v[32];
                        g_tmem_ld32(tmem_base + (unsigned)(acc * GM + c0 + h * 32) + ((unsigned)(quad * 32) << 16), v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (rows_here < 64) {  // the corpus ends inside this tile: rows that do not exist never pass
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (h * 32 + j >= rows_here) v[j] = -(1 << 30);
                        }
                        // first test, branch-free: ts - v - 1 is negative exactly when v >= ts (both are far
                        // from the ends of the int range), so the sign of an OR says "some row passes";
                        // four ORs over 8 rows each, so that a thread with a hit looks at 8 rows, not 32
                        int any[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int j = 0; j < 32; ++j) any[j >> 3] |= ts - v[j] - 1;
                        if ((any[0] | any[1] | any[2] | any[3]) < 0) {
                            const unsigned base_slot = (unsigned)(row0 + h * 32);
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                if (any[g] < 0) {
                                    // which of the 8 rows pass, as bits (straight-line code), then one turn of
                                    // the loop per passing row: rows that fail cost two instructions each
                                    unsigned m = 0u;
#pragma unroll
                                    for (int jj = 0; jj < 8; ++jj) m |= (v[8 * g + jj] >= ts) ? (1u << jj) : 0u;
                                    while (m != 0u) {
                                        const int jj = __ffs(m) - 1;
                                        m &= m - 1u;
                                        const int a0 = (jj & 1) ? v[8 * g + 1] : v[8 * g + 0], a1 = (jj & 1) ? v[8 * g + 3] : v[8 * g + 2];
                                        const int a2 = (jj & 1) ? v[8 * g + 5] : v[8 * g + 4], a3 = (jj & 1) ? v[8 * g + 7] : v[8 * g + 6];
                                        const int b0 = (jj & 2) ? a1 : a0, b1 = (jj & 2) ? a3 : a2;
                                        const int sc = (jj & 4) ? b1 : b0;
                                        const unsigned long long key = make_key(ord_from_i32(sc), base_slot + (unsigned)(8 * g + jj));
                                        if (key > thr) __stcg(my_list + cnt++, key);
                                    }
                                }
                            }
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) g_mbar_arrive_leader(&ctl->tmem_empty[acc]);  // the leader's MMAs may overwrite it
                }
                if (++acc == GACC) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
                // One meeting per tile and quad: its barrier ORs "one of our lists needs a cut".
                int prune;
                asm volatile(
                    "{\n\t.reg .pred p, r;\n\t"
                    "setp.gt.s32 p, %1, %3;\n\t"
                    "bar.red.or.pred r, %2, 128, p;\n\t"
                    "selp.s32 %0, 1, 0, r;\n\t}"
                    : "=r"(prune)
                    : "r"(cnt), "r"(qbar), "r"(GSUB_LIMIT)
                    : "memory");
                ok = ctl->epilogue_failed == 0;
                if (!ok) break;
                const bool refresh = (step & 15) == 15;  // look at the other pairs' thresholds now and then
                if (prune || refresh) {
                    if (prune) {
                        ctl->cnt4[q][part] = cnt;
                        __threadfence();
                        asm volatile("bar.sync %0, 128;" ::"r"(qbar) : "memory");
                        // every query of the quad is cut, not only the full ones: the queries fill at similar
                        // rates, so this turns many one-list stalls into few events with all four warps at work
                        for (int qq = quad * 32 + part; qq < quad * 32 + 32; qq += GPARTS) {
                            g_prune_query(ctl, cand + (size_t)qq * GCAP_MAX, qq, a.k, lane);
                            if (lane == 0 && q0 + qq < a.nq) atomicMax(gthr + qq, ctl->thr[qq]);
                        }
                        asm volatile("bar.sync %0, 128;" ::"r"(qbar) : "memory");
                        cnt = ctl->cnt4[q][part];
                    }
                    // a key below another pair's k-th best cannot be among the k best overall
                    if (part == 0 && q0 + q < a.nq) {
                        const unsigned long long g = __ldcg(gthr + q);
                        if (g > ctl->thr[q]) {
                            ctl->thr[q] = g;
                            ctl->thr_score[q] = i32_from_ord(key_ord(g));
                        }
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(qbar) : "memory");
                    ts = ctl->thr_score[q];
                    thr = ctl->thr[q];
                }
            }
            ctl->cnt4[q][part] = cnt;
            // final lists of this segment: [slice][query][k], ranked; as many warps sort as the scratch has room for
            asm volatile("bar.sync 5, 512;" ::: "memory");
            __threadfence();
            int ksz = 2;
            while (ksz < a.k) ksz <<= 1;
            const int sorters = min(GEPI_WARPS, GSORT_BYTES / (ksz * 8));
            unsigned long long *scratch = sm_sort + (size_t)ew * ksz;
            for (int qq = ew; ew < sorters && qq < GN; qq += sorters) {
                if (q0 + qq >= a.nq) continue;
                const unsigned long long *cq = cand + (size_t)qq * GCAP_MAX;
                int total = 0;
#pragma unroll
                for (int p = 0; p < GPARTS; ++p) total += ctl->cnt4[qq][p];
                if (total > a.k) {  // cut to the best k, dealt out over the four lists
                    g_prune_query(ctl, cand + (size_t)qq * GCAP_MAX, qq, a.k, lane);
                    for (int j = lane; j < ksz; j += 32) scratch[j] = (ok && j < a.k) ? g_dealt_key(cq, j) : 0ull;
                } else {            // fewer than k in all: take the lists as they are
                    for (int j = lane; j < ksz; j += 32) scratch[j] = 0ull;
                    __syncwarp();
                    int at = 0;
                    for (int p = 0; p < GPARTS; ++p) {
                        const int c = ctl->cnt4[qq][p];
                        for (int j = lane; ok && j < c; j += 32) scratch[at + j] = __ldcg(cq + p * GSUB + j);
                        at += c;
                    }
                }
                __syncwarp();
                g_warp_sort_desc(scratch, ksz, lane);
                unsigned long long *dst = a.lists + ((size_t)sg.slice * a.nq + (q0 + qq)) * a.k;
                for (int j = lane; j < a.k; j += 32) dst[j] = scratch[j];
                __syncwarp();
            }
            asm volatile("bar.sync 5, 512;" ::: "memory");
        }
    }
    // ------------------------------ teardown ------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && ctl->failed != 0) {
        if (a.error != nullptr) atomicExch(a.error, 1);
        // copies this CTA issued may still be landing in its shared memory: give them time before it is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {}
    }
    g_pair_sync();  // nothing of the partner is still aimed at this CTA's barriers or tensor memory
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(GACC * GM) : "memory");
    }
}

}  // namespace lk

namespace lk {

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_fn get_encode() {
    static encode_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_fn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// [rows x ld bytes] row-major int8 matrix, boxes of box_rows rows x 128 bytes, 128-byte swizzle;
// out-of-range rows and columns read as zero.
static int make_map(CUtensorMap *tm, const void *base, long long rows, long long ld, int box_rows) {
    encode_fn enc = get_encode();
    if (!enc) return fail(LK_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)ld, (cuuint64_t)std::max<long long>(rows, 1)};
    const cuuint64_t strides[1] = {(cuuint64_t)ld};
    const cuuint32_t box[2] = {(cuuint32_t)GSLICE, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LK_ECUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return 0;
}


bool gemm_supported(long long ld, int k) { return ld % 16 == 0 && ld <= 1152 && k >= 1 && k <= GEMM_MAX_K; }

// CTAs of the launch: pairs of SMs.
static int gemm_grid(int sm_count) { return std::max(2, sm_count & ~1); }

// per CTA: 128 candidate lists
size_t gemm_cand_bytes(int sm_count) { return (size_t)gemm_grid(sm_count) * GN * GCAP_MAX * 8; }
// one shared threshold per query, rounded up to whole 256-query tiles; the caller clears it before a launch
size_t gemm_thr_bytes(int nq) { return (size_t)((nq + 2 * GN - 1) / (2 * GN)) * 2 * GN * 8; }

// Most result lists one query tile ends up with: its dedicated pairs plus the floaters whose runs touch it.
int gemm_max_slices(int sm_count, int nq, long long n) {
    const int pairs = gemm_grid(sm_count) / 2;
    const int qtiles = (nq + 2 * GN - 1) / (2 * GN);
    const GemmSplit sp = gemm_split(pairs, qtiles, std::max<long long>(1, (n + GM - 1) / GM));
    int most = 0;
    if (sp.units > 0)
        for (int qt = 0; qt < qtiles; ++qt) {
            const int first = gemm_float_owner(sp, (long long)qt * sp.tail);
            const int last = gemm_float_owner(sp, (long long)(qt + 1) * sp.tail - 1);
            most = std::max(most, last - first + 1);
        }
    return std::max(1, sp.D + most);
}

// Enqueue the batched search: lists[slice][nq][k] receives the ranked keys of every pair that
// worked on a query's tile (unused slices stay as the caller cleared them: zero).
int gemm_launch(const unsigned char *d_rows, long long n, long long ld, const unsigned char *d_queries, int nq, int k,
                unsigned long long *d_cand, unsigned long long *d_gthr, unsigned long long *d_lists, int *d_error,
                int sm_count, cudaStream_t stream, long long *launches) {
    CUtensorMap tm_rows, tm_q;
    LK_TRY(make_map(&tm_rows, d_rows, n, ld, GR));
    LK_TRY(make_map(&tm_q, d_queries, nq, ld, GN));
    const int ks = (int)((ld + GSLICE - 1) / GSLICE);
    const size_t fixed = (size_t)ks * GQ_SLICE_BYTES + GSORT_BYTES + sizeof(GemmShared) + 1024;
    int stages = (int)((226 * 1024 - fixed) / GSLICE_BYTES);
    stages = std::min(stages, 8);
    if (stages < 2) return fail(LK_ERANGE, "gemm search: rows too wide for the resident query tile");
    const size_t smem = fixed + (size_t)stages * GSLICE_BYTES;
    cudaError_t e = cudaFuncSetAttribute((const void *)k_gemm_i8_topk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(LK_ECUDA, std::string("gemm attr: ") + cudaGetErrorString(e));
    GemmArgs a;
    a.n = n;
    a.nq = nq;
    a.ks = ks;
    a.stages = stages;
    a.k = k;
    a.qtiles = (nq + 2 * GN - 1) / (2 * GN);
    a.cand = d_cand;
    a.gthr = d_gthr;
    a.lists = d_lists;
    a.error = d_error;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gemm_grid(sm_count));
    cfg.blockDim = dim3(GTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;  // the two CTAs of a pair share their MMAs
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, k_gemm_i8_topk, tm_rows, tm_q, a);
    if (e != cudaSuccess) return fail(LK_ECUDA, std::string("gemm launch: ") + cudaGetErrorString(e));
    if (launches) ++*launches;
    return 0;
}

}  // namespace lk
