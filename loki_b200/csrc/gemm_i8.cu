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
// Shape of one CTA (576 threads, one CTA per SM):
//   warp 0     TMA producer: 2-D tiled loads (128-byte swizzle) of corpus tiles
//              [256 rows x 128 K-bytes] into a ring of stages; loads the CTA's query
//              tile [128 queries x all K] once, it stays resident in shared memory
//   warp 1     allocates tensor memory and issues the MMAs: D[128 queries x 256 rows]
//              += Q[128 x 32] * R[256 x 32]^T, four per 128-byte K slice (the queries are the
//              M side, so that every instruction carries N = 256: 128 x 256 x 32 per issue);
//              commits free the stage / publish the accumulator through mbarriers.  Both
//              single-thread roles run their loops warp-wide and let an elected lane issue.
//   warps 2-17 epilogue: a tensor-memory lane is a query, a column a corpus row: a thread
//              reads its query's scores of 64 rows per tile, tests them against the query's
//              threshold (one register) with one add and half an OR each, and appends the few
//              survivors to its query's candidate list; two accumulator buffers (all 512
//              columns of tensor memory) let the next tile's MMAs run meanwhile.  A list that
//              fills up is cut back to its best k by a warp-wide selection (bisection on the
//              score with the keys in registers), which also raises the query's threshold;
//              lists are sorted once, at the end.
// A CTA owns one tile of 128 queries and every ns-th corpus tile; the CTAs of one query
// tile split the corpus between them and their lists are merged by k_merge_lists.
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

constexpr int GN = 128;            // queries per tile (MMA M, tensor-memory lanes)
constexpr int GM = 256;            // corpus rows per tile (MMA N, tensor-memory columns)
constexpr int GSLICE = 128;        // K bytes per shared-memory slice: one swizzle row
constexpr int GQ_SLICE_BYTES = GN * GSLICE;  // 16 KB: one K slice of the 128-query tile
constexpr int GSLICE_BYTES = GM * GSLICE;    // 32 KB: one K slice of a 256-row corpus tile
constexpr int GCAP_MAX = 1024;     // most candidate keys a query holds between prunes (k <= 256)
constexpr int GEPI_WARPS = 16;     // epilogue warps: four per tensor-memory lane quadrant, 32 queries each
constexpr int GEPI_THREADS = GEPI_WARPS * 32;
constexpr int GTHREADS = 64 + GEPI_THREADS;
constexpr int GACC = 2;            // accumulators in tensor memory: 2 x 256 columns = all 512
// A query's list holds GCAP_MAX keys.  One tile adds at most 256 to a list; the check that
// triggers a cut may miss what other warps append while it runs, so it leaves room for two
// tiles: a list is cut back to k whenever it exceeds cap - 512, i.e. after at least
// 512 - k new survivors.
__host__ __device__ inline int gemm_cap(int) { return GCAP_MAX; }
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
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(g_smem(bar)), "r"(parity)
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
// 2-D tiled TMA load: box at (x = byte column, y = row) of the tensor map -> shared memory
__device__ __forceinline__ void g_tma_load_2d(void *dst, const CUtensorMap *tm, int x, int y, unsigned long long *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            g_smem(dst)),
        "l"(reinterpret_cast<unsigned long long>(tm)), "r"(x), "r"(y), "r"(g_smem(bar))
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
// Instruction descriptor: int8 x int8 (both signed, K-major) -> int32, M = 128 queries, N = 256 rows.
constexpr unsigned G_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(GM >> 3) << 17) | ((unsigned)(GN >> 4) << 24);

__device__ __forceinline__ void g_mma_i8(unsigned tmem_d, unsigned long long da, unsigned long long db, bool accumulate) {
    const unsigned acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(da), "l"(db), "r"(G_IDESC), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void g_mma_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(g_smem(bar)) : "memory");
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

// Which query tile and which share of the corpus tiles a CTA owns: `grid` CTAs are dealt
// out to `qtiles` query tiles as evenly as possible (the first grid % qtiles tiles get one more).
__host__ __device__ inline void gemm_assign(int cta, int grid, int qtiles, int *qt, int *slice, int *nslices) {
    const int base = grid / qtiles, rem = grid % qtiles;
    if (cta < rem * (base + 1)) {
        *qt = cta / (base + 1);
        *slice = cta % (base + 1);
        *nslices = base + 1;
    } else {
        const int c = cta - rem * (base + 1);
        *qt = rem + c / base;
        *slice = c % base;
        *nslices = base;
    }
}

#ifdef LK_GEMM_PROFILE
__device__ unsigned long long g_gemm_prof[16];  // summed clocks per role and phase (tuning builds only)
#define GPROF_T0 const long long _pt0 = clock64()
#define GPROF_ADD(i) atomicAdd(&g_gemm_prof[i], (unsigned long long)(clock64() - _pt0))
#else
#define GPROF_T0
#define GPROF_ADD(i)
#endif

struct GemmShared {  // control words behind the data regions
    unsigned long long full[8], empty[8], b_full, tmem_full[GACC], tmem_empty[GACC];
    unsigned long long thr[GN];  // per query: keys must exceed this to enter its list
    alignas(16) int thr_score[GN];  // score part of thr: the cheap first test (score >= thr_score)
    int cnt[GN];                 // per query: keys in its list
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
    const int n = min(ctl->cnt[q], KPL * 32);
    if (n <= k) return;
    unsigned hi[KPL], lo[KPL];  // score word (0 = no key: below every real one) and slot word
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        const int i = lane + 32 * u;
        const unsigned long long key = (i < n) ? __ldcg(cand_q + i) : 0ull;
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
    // X = the largest score word x with count(hi >= x) >= k;  count(hi >= mn) = n > k
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
    // compaction: lane-local count, exclusive scan over lanes, stores behind all loads
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
        if (keep) __stcg(cand_q + pos++, ((unsigned long long)hi[u] << 32) | lo[u]);
    }
    __syncwarp();
    if (lane == 0) {
        ctl->cnt[q] = k;
        const unsigned long long kth = ((unsigned long long)X << 32) | ymin;  // the smallest key kept
        if (kth > ctl->thr[q]) {
            ctl->thr[q] = kth;
            ctl->thr_score[q] = i32_from_ord(X);
        }
    }
    __syncwarp();
}

__device__ inline void g_prune_query(GemmShared *ctl, unsigned long long *cand_q, int q, int k, int, int lane) {
    g_select_query<GCAP_MAX / 32>(ctl, cand_q, q, k, lane);
}

__global__ void __launch_bounds__(GTHREADS, 1)
k_gemm_i8_topk(const __grid_constant__ CUtensorMap tm_rows, const __grid_constant__ CUtensorMap tm_queries,
               const GemmArgs a) {
    extern __shared__ unsigned char g_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address
    unsigned char *smem = g_raw + ((1024u - (g_smem(g_raw) & 1023u)) & 1023u);
    unsigned char *sm_b = smem;                                        // [ks][128 queries][128 B]: the MMA's A operand
    unsigned char *sm_a = sm_b + (size_t)a.ks * GQ_SLICE_BYTES;        // [stages][256 rows][128 B]: the MMA's B operand
    const int cap = gemm_cap(a.k), limit = cap - 2 * GM;
    GemmShared *ctl = reinterpret_cast<GemmShared *>(sm_a + (size_t)a.stages * GSLICE_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int qt, slice, nslices;
    gemm_assign((int)blockIdx.x, (int)gridDim.x, a.qtiles, &qt, &slice, &nslices);
    qt += a.qtile0;
    const long long n_tiles = (a.n + GM - 1) / GM;
    const int q0 = qt * GN;  // first query of this CTA's tile

    if (tid == 0) {
        for (int i = 0; i < a.stages; ++i) {
            g_mbar_init(&ctl->full[i], 1);
            g_mbar_init(&ctl->empty[i], 1);
        }
        g_mbar_init(&ctl->b_full, 1);
        for (int i = 0; i < GACC; ++i) {
            g_mbar_init(&ctl->tmem_full[i], 1);
            g_mbar_init(&ctl->tmem_empty[i], GEPI_WARPS);  // one arrival per epilogue warp
        }
        ctl->failed = 0;
        ctl->epilogue_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < GN) {
        const bool live = q0 + tid < a.nq;  // queries past the end accept nothing
        ctl->thr[tid] = live ? 0ull : ~0ull;
        ctl->thr_score[tid] = live ? -(1 << 30) : (1 << 30);  // every real score is far inside +-2^30
        ctl->cnt[tid] = 0;
    }
    if (warp == 1) {  // tensor memory: GACC accumulators x 256 columns
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(g_smem(&ctl->tmem_base)),
                     "r"(GACC * GM)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = ctl->tmem_base;
    volatile int *failed = &ctl->failed;

    // The two single-thread roles run their loops with the whole warp (uniform control flow,
    // warp-uniform values: loop state and descriptors can live in uniform registers, which the
    // TMA and MMA instructions take their operands from) and let one elected lane issue.
    // With the loops inside `if (lane == 0)` every MMA cost about 155 clocks to issue, more than
    // twice what the tensor pipe needs to execute it.
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (g_elect_one()) {
            g_mbar_expect_tx(&ctl->b_full, (unsigned)(a.ks * GQ_SLICE_BYTES));
            for (int s = 0; s < a.ks; ++s)
                g_tma_load_2d(sm_b + (size_t)s * GQ_SLICE_BYTES, &tm_queries, s * GSLICE, q0, &ctl->b_full);
        }
        __syncwarp();
        int stage = 0;
        unsigned phase = 0;
        bool ok = true;
        for (long long t = slice; ok && t < n_tiles; t += nslices) {
            for (int s = 0; s < a.ks; ++s) {
                { GPROF_T0; ok = g_mbar_wait_warp(&ctl->empty[stage], phase ^ 1u, failed); if (lane == 0) GPROF_ADD(0); }
                if (!ok) break;
                if (g_elect_one()) {
                    g_mbar_expect_tx(&ctl->full[stage], (unsigned)GSLICE_BYTES);
                    g_tma_load_2d(sm_a + (size_t)stage * GSLICE_BYTES, &tm_rows, s * GSLICE, (int)(t * GM),
                                  &ctl->full[stage]);
                }
                __syncwarp();
                if (++stage == a.stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        bool ok = g_mbar_wait_warp(&ctl->b_full, 0u, failed);
        const unsigned long long da0 = g_smem_desc(g_smem(sm_a)), db0 = g_smem_desc(g_smem(sm_b));
        int stage = 0, acc = 0;
        unsigned phase = 0, acc_phase = 0;
        for (long long t = slice; ok && t < n_tiles; t += nslices) {
            { GPROF_T0; ok = g_mbar_wait_warp(&ctl->tmem_empty[acc], acc_phase ^ 1u, failed); if (lane == 0) GPROF_ADD(1); }
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned d = tmem_base + (unsigned)(acc * GM);
            for (int s = 0; s < a.ks; ++s) {
                { GPROF_T0; ok = g_mbar_wait_warp(&ctl->full[stage], phase, failed); if (lane == 0) GPROF_ADD(2); }
                if (!ok) break;
                // (no tcgen05 fence here: the stage was filled by TMA, whose completion on the mbarrier
                // orders it for the MMAs; a fence per slice drained the MMA queue at every slice)
                // the start-address field counts 16-byte units: one slice further = + 1024
                const unsigned long long da = da0 + (unsigned long long)(stage * (GSLICE_BYTES >> 4));     // corpus rows
                const unsigned long long db = db0 + (unsigned long long)(s * (GQ_SLICE_BYTES >> 4));      // queries
                if (g_elect_one()) {
#pragma unroll
                    for (int k4 = 0; k4 < GSLICE / 32; ++k4)  // 32 K-bytes per MMA: +2 in 16-byte units
                        g_mma_i8(d, db + (unsigned long long)(2 * k4), da + (unsigned long long)(2 * k4), (s | k4) != 0);
                    g_mma_commit(&ctl->empty[stage]);  // the stage is free once these MMAs have read it
                }
                __syncwarp();
                if (++stage == a.stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) break;
            if (g_elect_one()) g_mma_commit(&ctl->tmem_full[acc]);  // accumulator complete
            __syncwarp();
            if (++acc == GACC) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        // 16 warps.  A tensor-memory lane is a query, a column a corpus row of the tile.  A warp may
        // read the lanes 32 * (warp % 4) .. + 31 (the hardware's rule), i.e. 32 queries, and takes
        // one quarter of the 256 columns: one query x 64 corpus rows per thread and tile, so the
        // threshold is one register and every survivor of a thread goes to the thread's own query.
        const int ew = warp - 2;       // 0..15
        const int quad = warp & 3;
        const int c0 = (ew >> 2) * 64;
        const int etid = ew * 32 + lane;
        const int q = quad * 32 + lane;  // this thread's query within the tile
        unsigned long long *cand = a.cand + (size_t)blockIdx.x * GN * GCAP_MAX;
        unsigned long long *my_list = cand + (size_t)q * GCAP_MAX;
        int acc = 0;
        unsigned acc_phase = 0;
        bool ok = true;
        for (long long t = slice; t < n_tiles; t += nslices) {
            bool have;
            { GPROF_T0; have = g_mbar_wait_warp(&ctl->tmem_full[acc], acc_phase, failed); if (etid == 0) GPROF_ADD(3); }
            GPROF_T0;
            if (!have) ctl->epilogue_failed = 1;  // read by all epilogue threads behind the barrier below
            if (have) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int ts = ctl->thr_score[q];
                const long long row0 = t * GM + c0;
                const int rows_here = (int)min((long long)64, a.n - row0);  // columns past the corpus hold zeros
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    int v[32];
                    g_tmem_ld32(tmem_base + (unsigned)(acc * GM + c0 + h * 32) + ((unsigned)(quad * 32) << 16), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    // first test, branch-free: ts - v - 1 is negative exactly when v >= ts (both are far
                    // from the ends of the int range), so the sign of the OR says "some row passes"
                    int any = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) any |= ts - v[j] - 1;
                    if (any < 0) {  // rare once the threshold has risen
                        const unsigned long long thr = ctl->thr[q];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (v[j] >= ts && h * 32 + j < rows_here) {
                                const unsigned long long key = make_key(ord_from_i32(v[j]), (unsigned)(row0 + h * 32 + j));
                                if (key > thr) {
                                    const int pos = atomicAdd(&ctl->cnt[q], 1);
                                    if (pos < cap) __stcg(my_list + pos, key);
                                }
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) g_mbar_arrive(&ctl->tmem_empty[acc]);
            }
            if (etid == 0) GPROF_ADD(4);
            if (++acc == GACC) {
                acc = 0;
                acc_phase ^= 1u;
            }
            // One barrier per tile: it also ORs "one of my lists passed the mark".  The count a
            // thread reads may miss appends of warps still working on this tile; the mark
            // leaves room for that (see gemm_cap) and the next tile's check sees them.
            const int over = (etid < GN && ctl->cnt[etid] > limit) ? 1 : 0;
            int prune;
            asm volatile(
                "{\n\t.reg .pred p, r;\n\t"
                "setp.ne.s32 p, %1, 0;\n\t"
                "bar.red.or.pred r, 1, 512, p;\n\t"
                "selp.s32 %0, 1, 0, r;\n\t}"
                : "=r"(prune)
                : "r"(over)
                : "memory");
            ok = ctl->epilogue_failed == 0;
            if (!ok) break;
            if (prune) {
                GPROF_T0;
                __threadfence();
                // every list above k is cut, not only the full ones: the queries of a tile fill at
                // similar rates, so this turns hundreds of one-list stalls into a handful of events
                // in which all warps work at once
                for (int q = ew; q < GN; q += GEPI_WARPS)
                    if (ctl->cnt[q] > a.k) g_prune_query(ctl, cand + (size_t)q * GCAP_MAX, q, a.k, cap, lane);
                asm volatile("bar.sync 1, 512;" ::: "memory");
                if (etid == 0) GPROF_ADD(5);
            }
        }
        // final lists of this CTA: [slice][query][k], ranked.  The corpus stages are idle by now
        // (the last accumulator was complete before the last tile was read): they are the sort scratch.
        asm volatile("bar.sync 1, 512;" ::: "memory");
        __threadfence();
        int ksz = 2;
        while (ksz < a.k) ksz <<= 1;
        const int sorters = min(GEPI_WARPS, (int)((size_t)a.stages * GSLICE_BYTES / ((size_t)ksz * 8)));
        if (ew < sorters) {
            unsigned long long *scratch = reinterpret_cast<unsigned long long *>(sm_a) + (size_t)ew * ksz;
            for (int q = ew; q < GN; q += sorters) {
                if (q0 + q >= a.nq) continue;
                g_prune_query(ctl, cand + (size_t)q * GCAP_MAX, q, a.k, cap, lane);
                const int keep = ok ? min(ctl->cnt[q], a.k) : 0;
                for (int i = lane; i < ksz; i += 32) scratch[i] = (i < keep) ? __ldcg(cand + (size_t)q * GCAP_MAX + i) : 0ull;
                __syncwarp();
                g_warp_sort_desc(scratch, ksz, lane);
                unsigned long long *dst = a.lists + ((size_t)slice * a.nq + (q0 + q)) * a.k;
                for (int i = lane; i < a.k; i += 32) dst[i] = scratch[i];
                __syncwarp();
            }
        }
    }
    // ------------------------------ teardown ------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && ctl->failed != 0 && a.error != nullptr) atomicExch(a.error, 1);
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(GACC * GM) : "memory");
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

#ifdef LK_GEMM_PROFILE
extern "C" __attribute__((visibility("default"))) void lk_debug_gemm_profile(unsigned long long *out16, int reset) {
    cudaMemcpyFromSymbol(out16, g_gemm_prof, sizeof(unsigned long long) * 16);
    if (reset) {
        unsigned long long z[16] = {};
        cudaMemcpyToSymbol(g_gemm_prof, z, sizeof(z));
    }
}
#endif

bool gemm_supported(long long ld, int k) { return ld % 16 == 0 && ld <= 1152 && k >= 1 && k <= GEMM_MAX_K; }

size_t gemm_cand_bytes(int grid) { return (size_t)grid * GN * GCAP_MAX * 8; }

int gemm_max_slices(int grid, int nq) {
    const int qtiles = (nq + GN - 1) / GN;
    const int per_launch = std::min(qtiles, grid);
    return grid / per_launch + (grid % per_launch ? 1 : 0);
}

// Enqueue the batched search: lists[slice][nq][k] receives every CTA's ranked keys.
int gemm_launch(const unsigned char *d_rows, long long n, long long ld, const unsigned char *d_queries, int nq, int k,
                unsigned long long *d_cand, unsigned long long *d_lists, int *d_error, int sm_count,
                cudaStream_t stream, long long *launches) {
    CUtensorMap tm_rows, tm_q;
    LK_TRY(make_map(&tm_rows, d_rows, n, ld, GM));
    LK_TRY(make_map(&tm_q, d_queries, nq, ld, GN));
    const int ks = (int)((ld + GSLICE - 1) / GSLICE);
    const size_t fixed = (size_t)ks * GQ_SLICE_BYTES + sizeof(GemmShared) + 1024;
    int stages = (int)((224 * 1024 - fixed) / GSLICE_BYTES);
    stages = std::min(stages, 8);
    if (stages < 2) return fail(LK_ERANGE, "gemm search: rows too wide for the resident query tile");
    const size_t smem = fixed + (size_t)stages * GSLICE_BYTES;
    cudaError_t e = cudaFuncSetAttribute((const void *)k_gemm_i8_topk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(LK_ECUDA, std::string("gemm attr: ") + cudaGetErrorString(e));
    const int qtiles = (nq + GN - 1) / GN;
    for (int qt0 = 0; qt0 < qtiles; qt0 += sm_count) {  // at most one query tile per CTA and launch
        GemmArgs a;
        a.n = n;
        a.nq = nq;
        a.ks = ks;
        a.stages = stages;
        a.k = k;
        a.qtile0 = qt0;
        a.qtiles = std::min(qtiles - qt0, sm_count);
        a.cand = d_cand;
        a.lists = d_lists;
        a.error = d_error;
        k_gemm_i8_topk<<<sm_count, GTHREADS, smem, stream>>>(tm_rows, tm_q, a);
        e = cudaGetLastError();
        if (e != cudaSuccess) return fail(LK_ECUDA, std::string("gemm launch: ") + cudaGetErrorString(e));
        if (launches) ++*launches;
    }
    return 0;
}

}  // namespace lk
