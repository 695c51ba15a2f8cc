// Scoring scan: one query against N stored rows, fused with exact top-k selection.
//
// This is the device replacement for the reference's hot loop
//   scanTopK   media-server/embedindex/embedindex.go:424-457
//   Cosine     media-server/embedvec/embedvec.go:113-122   (float32 in, float64 accumulate)
//   centered   media-server/embedindex/embedindex.go:297-305
//   topK/sort  media-server/embedindex/embedindex.go:483-534
// plus the int8 variant this project defines (int8 x int8 -> int32, exact).
//
// The kernel is HBM-bound: every query streams the whole corpus once
// (rows x row-bytes), nothing else touches DRAM except k keys per CTA at the end.
//
// Work decomposition
//   * grid  = as many CTAs as are resident at once (a multiple of the SM count);
//             CTA c owns a contiguous range of 32-row batches;
//   * warp  = one batch of 32 consecutive rows at a time; within the warp, groups
//             of G lanes (G = 1..32, a power of two chosen from the row width)
//             share a row: lane l of a group reads 16-byte chunks l, l+G, ... of
//             the row, so a group reads 16*G contiguous bytes per instruction and
//             R rows are in flight per lane;
//   * each lane keeps one partial accumulator per row of its group; a transposed
//             butterfly (G-1 shuffles for G rows) leaves lane i with the finished
//             score of row i of the batch;
//   * the score becomes a 64-bit ranking key and is offered to the CTA's
//             candidate buffer (topk.cuh).
// Warps run free of each other; they meet at a barrier only when the candidate
// buffer is nearly full (to prune it) and when they run out of rows.
#include <cuda_fp16.h>

#include <algorithm>

#include "bulk.cuh"
#include "scan.cuh"
#include "topk.cuh"

namespace lk {

// ---------------------------------------------------------------------------
// Per-storage-type arithmetic
// ---------------------------------------------------------------------------

struct TraitsI8 {
    using acc_t = int;
    static constexpr int kRows = 8;        // rows in flight per lane group
    static constexpr int kQBytes = 16;     // shared-memory query bytes per chunk
    // query in shared memory: the int8 codes as they are
    __device__ static void stage_query(unsigned char *qs, const unsigned char *q, int chunks) {
        const int4 *src = reinterpret_cast<const int4 *>(q);
        int4 *dst = reinterpret_cast<int4 *>(qs);
        for (int j = threadIdx.x; j < chunks; j += blockDim.x) dst[j] = src[j];
    }
    struct QChunk { int4 q; };
    __device__ __forceinline__ static QChunk load_q(const unsigned char *qs, int j, int) {
        QChunk c;
        c.q = reinterpret_cast<const int4 *>(qs)[j];
        return c;
    }
    __device__ __forceinline__ static void dot(acc_t &acc, const int4 &v, const QChunk &c) {
        acc = __dp4a(v.x, c.q.x, acc);
        acc = __dp4a(v.y, c.q.y, acc);
        acc = __dp4a(v.z, c.q.z, acc);
        acc = __dp4a(v.w, c.q.w, acc);
    }
    __device__ __forceinline__ static acc_t shfl(acc_t v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
    __device__ __forceinline__ static uint32_t finish(acc_t acc, const ScanArgs &, unsigned) {
        return ord_from_i32(acc);
    }
};

struct TraitsF32 {
    using acc_t = double;
    static constexpr int kRows = 4;
    static constexpr int kQBytes = 32;
    // query in shared memory as float64, split in two planes so that consecutive
    // lanes read consecutive 16-byte words: plane A holds elements (4j, 4j+1),
    // plane B holds (4j+2, 4j+3) of chunk j.
    __device__ static void stage_query(unsigned char *qs, const unsigned char *q, int chunks) {
        const float4 *src = reinterpret_cast<const float4 *>(q);
        double2 *pa = reinterpret_cast<double2 *>(qs);
        double2 *pb = pa + chunks;
        for (int j = threadIdx.x; j < chunks; j += blockDim.x) {
            float4 f = src[j];
            pa[j] = make_double2((double)f.x, (double)f.y);
            pb[j] = make_double2((double)f.z, (double)f.w);
        }
    }
    struct QChunk { double2 a, b; };
    __device__ __forceinline__ static QChunk load_q(const unsigned char *qs, int j, int chunks) {
        QChunk c;
        const double2 *pa = reinterpret_cast<const double2 *>(qs);
        c.a = pa[j];
        c.b = pa[chunks + j];
        return c;
    }
    // float32 x float32 products are exact in float64, so fma here equals the
    // reference's multiply-then-add; only the order of the additions differs.
    __device__ __forceinline__ static double widen(int b) { return (double)__int_as_float(b); }
    __device__ __forceinline__ static void dot(acc_t &acc, const int4 &v, const QChunk &c) {
        acc = fma(widen(v.x), c.a.x, acc);
        acc = fma(widen(v.y), c.a.y, acc);
        acc = fma(widen(v.z), c.b.x, acc);
        acc = fma(widen(v.w), c.b.y, acc);
    }
    __device__ __forceinline__ static acc_t shfl(acc_t v, int m) {
        return __longlong_as_double((long long)shfl_xor_u64((uint64_t)__double_as_longlong(v), m));
    }
    __device__ __forceinline__ static uint32_t finish(acc_t acc, const ScanArgs &a, unsigned slot) {
        float s = (float)acc;  // the single rounding of embedvec.Cosine
        if (a.cnorm != nullptr) {
            const float cn = a.cnorm[slot];
            s = (cn < 1e-6f) ? 0.0f : __fdiv_rn(__fsub_rn(s, a.cq), cn);
        }
        return ord_from_f32(s);
    }
};

struct TraitsF16 {
    using acc_t = float;
    static constexpr int kRows = 8;
    static constexpr int kQBytes = 32;
    // 8 halves per chunk; query kept as float32, two planes of 4 floats.
    __device__ static void stage_query(unsigned char *qs, const unsigned char *q, int chunks) {
        const float4 *src = reinterpret_cast<const float4 *>(q);
        float4 *pa = reinterpret_cast<float4 *>(qs);
        float4 *pb = pa + chunks;
        for (int j = threadIdx.x; j < chunks; j += blockDim.x) {
            pa[j] = src[2 * j];
            pb[j] = src[2 * j + 1];
        }
    }
    struct QChunk { float4 a, b; };
    __device__ __forceinline__ static QChunk load_q(const unsigned char *qs, int j, int chunks) {
        QChunk c;
        const float4 *pa = reinterpret_cast<const float4 *>(qs);
        c.a = pa[j];
        c.b = pa[chunks + j];
        return c;
    }
    __device__ __forceinline__ static void dot(acc_t &acc, const int4 &v, const QChunk &c) {
        const __half2 h0 = *reinterpret_cast<const __half2 *>(&v.x);
        const __half2 h1 = *reinterpret_cast<const __half2 *>(&v.y);
        const __half2 h2 = *reinterpret_cast<const __half2 *>(&v.z);
        const __half2 h3 = *reinterpret_cast<const __half2 *>(&v.w);
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        const float2 f2 = __half22float2(h2), f3 = __half22float2(h3);
        acc = fmaf(f0.x, c.a.x, acc);
        acc = fmaf(f0.y, c.a.y, acc);
        acc = fmaf(f1.x, c.a.z, acc);
        acc = fmaf(f1.y, c.a.w, acc);
        acc = fmaf(f2.x, c.b.x, acc);
        acc = fmaf(f2.y, c.b.y, acc);
        acc = fmaf(f3.x, c.b.z, acc);
        acc = fmaf(f3.y, c.b.w, acc);
    }
    __device__ __forceinline__ static acc_t shfl(acc_t v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
    __device__ __forceinline__ static uint32_t finish(acc_t acc, const ScanArgs &, unsigned) {
        return ord_from_f32(acc);
    }
};

// ---------------------------------------------------------------------------
// Result decoding shared by the scan's last CTA and the merge kernel
// ---------------------------------------------------------------------------
__device__ __forceinline__ void emit_hit(int type, unsigned long long key, int i, long long base,
                                         float dq, long long *out_ids, float *out_scores,
                                         int *out_iscores) {
    if (key == 0ull) {
        out_ids[i] = -1;
        out_scores[i] = 0.0f;
        if (out_iscores) out_iscores[i] = 0;
        return;
    }
    out_ids[i] = base + (long long)key_slot(key);
    if (type == SCAN_I8) {
        const int s = i32_from_ord(key_ord(key));
        out_scores[i] = (float)s * dq;
        if (out_iscores) out_iscores[i] = s;
    } else {
        out_scores[i] = f32_from_ord(key_ord(key));
        if (out_iscores) out_iscores[i] = 0;
    }
}

// ---------------------------------------------------------------------------
// One batch of (up to) 32 rows -> lane i holds the finished accumulator of row i.
// `row_ptr(i)` gives the address of batch row i (global or shared memory), `row_ok(i)`
// whether it exists; Load fetches 16 bytes from that address space.
// ---------------------------------------------------------------------------
struct LoadGlobal {
    __device__ __forceinline__ static int4 ld(const unsigned char *p) { return ld_stream16(p); }
};
struct LoadShared {
    __device__ __forceinline__ static int4 ld(const unsigned char *p) { return *reinterpret_cast<const int4 *>(p); }
};

// acc[t] += <row (grp*G + t) of the batch, query> over chunks [0, n_chunks) of the rows
// as laid out at row_ptr(i); q_chunk0 is the index of the first of those chunks in the query.
template <class TR, int G, int R, class Load, class RowPtr, class RowOk>
__device__ __forceinline__ void batch_accumulate(typename TR::acc_t (&acc)[G], const unsigned char *qs, int q_chunks,
                                                 int q_chunk0, int n_chunks, int lane, RowPtr row_ptr, RowOk row_ok) {
    const int grp = lane / G, gl = lane % G;
#pragma unroll
    for (int t0 = 0; t0 < G; t0 += R) {
        const unsigned char *p[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int in_batch = grp * G + t0 + r;
            ok[r] = row_ok(in_batch);
            p[r] = row_ptr(in_batch);
        }
#pragma unroll 2
        for (int j = gl; j < n_chunks; j += G) {
            const typename TR::QChunk qc = TR::load_q(qs, q_chunk0 + j, q_chunks);
            int4 v[R];
#pragma unroll
            for (int r = 0; r < R; ++r) v[r] = ok[r] ? Load::ld(p[r] + (size_t)j * 16) : make_int4(0, 0, 0, 0);
#pragma unroll
            for (int r = 0; r < R; ++r) TR::dot(acc[t0 + r], v[r], qc);
        }
    }
}

// transposed butterfly: lane i of the warp ends with the total of batch row i (in acc[0])
template <class TR, int G>
__device__ __forceinline__ typename TR::acc_t batch_reduce(typename TR::acc_t (&acc)[G], int lane) {
    using acc_t = typename TR::acc_t;
#pragma unroll
    for (int w = G / 2; w >= 1; w >>= 1) {
        const bool upper = (lane & w) != 0;
#pragma unroll
        for (int i = 0; i < w; ++i) {
            const acc_t send = upper ? acc[i] : acc[i + w];
            const acc_t keep = upper ? acc[i + w] : acc[i];
            acc[i] = keep + TR::shfl(send, w);
        }
    }
    return acc[0];
}

// Fixed-shape variant for the TMA-staged kernel: SC chunks per row slab and the row
// stride are compile-time, so every shared-memory load has an immediate offset and
// the whole batch unrolls; q[jj] is the query chunk for this lane's jj-th column.
template <class TR, int G, int SC>
__device__ __forceinline__ void slab_accumulate_fixed(typename TR::acc_t (&acc)[G],
                                                      const typename TR::QChunk (&q)[SC / G],
                                                      const unsigned char *stage, int lane) {
    constexpr int NJ = SC / G, W = SC * 16;
    const unsigned char *base = stage + (size_t)(lane / G) * G * W + (size_t)(lane % G) * 16;
#pragma unroll
    for (int t = 0; t < G; ++t) {
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) {
            const int4 v = *reinterpret_cast<const int4 *>(base + t * W + jj * G * 16);
            TR::dot(acc[t], v, q[jj]);
        }
    }
}

constexpr unsigned long long kPeerWaitNs = 2000000000ull;  // longest wait for another rank's list: 2 s

// Tag a rank stores into a slot's flag once its list for query `seq` is complete: never 0
// (the flags start at 0); the top bit says that the rank's own scan failed (a bounded wait
// ran out), which makes the query invalid on every rank.
constexpr unsigned kPeerPoison = 0x80000000u;
__device__ __forceinline__ unsigned peer_tag(unsigned seq) { return seq % 0x7ffffffeu + 1u; }

// Wait (bounded) until every rank's list for query `seq` has landed in this rank's inbox, merge
// them into `buf` and write the global result.  Called by all threads of one CTA.  Returns the
// number of hits, or -1 when a rank did not deliver in time or delivered a failed scan.
template <int TYPE>
__device__ __forceinline__ int peer_merge_emit(const PeerTable &pt, unsigned seq, int k, const CandBuf &buf,
                                               long long *out_ids, float *out_scores, int *out_iscores) {
    const int tid = threadIdx.x, T = blockDim.x;
    const int slot = (int)(seq % kPeerSlots);
    const unsigned want = peer_tag(seq);
    __shared__ int s_peer_bad;
    __syncthreads();
    if (tid == 0) s_peer_bad = 0;
    __syncthreads();
    if (tid < pt.world) {
        const unsigned int *f = &pt.inbox[pt.rank]->flags[slot][tid];
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == want) break;
            if (v == (want | kPeerPoison)) {
                s_peer_bad = 1;
                break;
            }
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > kPeerWaitNs) {  // a rank never delivered: give up, report, stay usable
                s_peer_bad = 1;
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
    const bool bad = s_peer_bad != 0;
    const PeerInbox *mine_in = pt.inbox[pt.rank];
    // When all ranks' lists fit twice into the buffer (a top-10 of 8 ranks: 80 keys) they are fetched in one
    // round trip, sorted in the lower half and kept as they came in the upper half, where the owner of
    // every hit is then found without further trips to memory.  Larger merges take the streaming path.
    const int total = pt.world * k, half = buf.cap >> 1;
    const bool local = total <= half;
    const unsigned long long *lists = buf.keys + half;  // [world][k], as delivered
    __shared__ int s_peer_cnt;
    if (local) {
        for (int i = tid; i < half; i += T) {
            const unsigned long long v = (i < total) ? __ldcg(&mine_in->keys[slot][i / k][i % k]) : 0ull;
            buf.keys[i] = v;
            buf.keys[half + i] = v;
        }
        if (tid == 0) {
            buf.ctrl->count = total;
            buf.ctrl->thr = 0ull;
            s_peer_cnt = 0;
        }
        __syncthreads();
        if (total <= T) {
            // a key per thread: its place is the number of keys above it (keys are distinct; 80 compares
            // against shared memory instead of a sorting network that this CTA runs once, from cold code)
            const unsigned long long mine = (tid < total) ? lists[tid] : 0ull;
            int above = 0;
            for (int j = 0; j < total; ++j) above += (lists[j] > mine) ? 1 : 0;
            const int present = __syncthreads_count(mine != 0ull);
            for (int i = tid; i < half; i += T) buf.keys[i] = 0ull;
            __syncthreads();
            if (mine != 0ull && above < k) buf.keys[above] = mine;
            if (tid == 0) s_peer_cnt = min(present, k);
        } else {
            cand_prune(buf);  // ranked, best k kept (empty entries are 0 and sort last)
            for (int i = tid; i < k; i += T)
                if (buf.keys[i] != 0ull && (i + 1 == k || buf.keys[i + 1] == 0ull)) s_peer_cnt = i + 1;
        }
        __syncthreads();
    } else {
        cand_select_from_lists(buf, &mine_in->keys[slot][0][0], pt.world, kPeerMaxK);
    }
    const int cnt = local ? s_peer_cnt : buf.ctrl->count;
    for (int i = tid; i < k; i += T) {
        const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
        if (key == 0ull) {
            emit_hit(TYPE, 0ull, i, 0, 0.0f, out_ids, out_scores, out_iscores);
            continue;
        }
        out_ids[i] = (long long)key_slot(key);  // already a global row number
        if (TYPE != SCAN_I8) {
            out_scores[i] = f32_from_ord(key_ord(key));
            if (out_iscores) out_iscores[i] = 0;
            continue;
        }
        // the float score was finished by the shard owning the row: find the key in the lists
        float sc = 0.0f;
        bool found = false;
        for (int r = 0; r < pt.world && !found; ++r) {
            int lo = 0, hi = k - 1;
            while (lo <= hi) {  // ranked descending
                const int mid = (lo + hi) >> 1;
                const unsigned long long v = local ? lists[r * k + mid] : __ldcg(&mine_in->keys[slot][r][mid]);
                if (v == key) {
                    sc = __ldcg(&mine_in->payload[slot][r][mid]);
                    found = true;
                    break;
                }
                if (v > key) lo = mid + 1; else hi = mid - 1;
            }
        }
        out_scores[i] = sc;
        if (out_iscores) out_iscores[i] = i32_from_ord(key_ord(key));
    }
    __syncthreads();
    return bad ? -1 : cnt;
}

// Shared tail of both scan kernels: publish this CTA's list; the last CTA to arrive
// merges all lists and writes the result.
// `spare` / `spare_keys`: shared memory the CTA no longer needs once it is out of rows (the
// streaming kernels' stage buffers).  The last CTA merges there when k is large: the keys above the
// merge's starting threshold number between k and a few k, and the CTA's own buffer (sized for k plus
// one round of appends) would often overflow, which costs a second, slower pass.
template <int TYPE>
__device__ __forceinline__ void publish_and_finish(const ScanArgs &a, const CandBuf &own, int *s_last,
                                                   unsigned long long *spare = nullptr, int spare_keys = 0) {
    const int tid = threadIdx.x, T = blockDim.x;
    unsigned long long *mine = a.part + (size_t)blockIdx.x * a.k;
    for (int i = tid; i < a.k; i += T) mine[i] = own.keys[i];
    if (tid == 0 && a.part_cnt != nullptr) a.part_cnt[blockIdx.x] = min(own.ctrl->count, a.k);
    __threadfence();
    __syncthreads();
    if (tid == 0) *s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    CandBuf buf = own;
    if (a.k > 32 && spare != nullptr) {
        int want = own.cap;
        while (want < 4 * a.k && want * 2 <= spare_keys) want <<= 1;
        if (want > own.cap) {
            buf.keys = spare;
            buf.cap = want;
            buf.limit = want - kScanThreads;
        }
    }
    if (a.k <= 32 && (int)(blockDim.x >> 5) * 32 <= buf.cap)
        cand_select_small(buf, a.part, (int)gridDim.x);
    else if (!cand_select_flat(buf, a.part, a.part_cnt, (int)gridDim.x))
        cand_select_from_lists(buf, a.part, (int)gridDim.x);
    int cnt = buf.ctrl->count;
    // a CTA whose bounded wait ran out has raised the flag before publishing its list
    const bool scan_bad = a.error != nullptr && *(volatile int *)a.error != 0;
    int *count_to = a.out_count;
    if (a.peer == nullptr) {
        for (int i = tid; i < a.k; i += T) {
            const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
            a.out_keys[i] = key;
            float dq = 0.0f;
            if (TYPE == SCAN_I8 && key != 0ull) dq = a.qscale * a.scales[key_slot(key)];
            emit_hit(TYPE, key, i, a.shard_base, dq, a.out_ids, a.out_scores, a.out_iscores);
        }
        if (scan_bad) cnt = -1;
    } else {
        // ---- sharded index: exchange with the other GPUs of the box, then merge ----
        // This shard's ranked list goes straight into every rank's inbox over NVLink
        // (plain stores to peer memory), followed by a release of the slot's flag.  Then this
        // CTA waits (bounded) until all ranks' lists for the query it is to merge have landed
        // in its own inbox and merges them.  No collective launch, no host round trip.
        const PeerTable &pt = *a.peer;
        const int slot = (int)(a.seq % kPeerSlots);
        const unsigned tag = peer_tag(a.seq) | (scan_bad ? kPeerPoison : 0u);
        for (int i = tid; i < a.k; i += T) {
            const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
            a.out_keys[i] = key;
            float pay = 0.0f;
            if (TYPE == SCAN_I8 && key != 0ull)
                pay = (float)i32_from_ord(key_ord(key)) * (a.qscale * a.scales[key_slot(key)]);
            // the low word holds ~row: subtracting the shard base adds it to the row number
            const unsigned long long gkey = key ? key - (unsigned long long)pt.base : 0ull;
            for (int r = 0; r < pt.world; ++r) {
                pt.inbox[r]->keys[slot][pt.rank][i] = gkey;
                if (TYPE == SCAN_I8) pt.inbox[r]->payload[slot][pt.rank][i] = pay;
            }
        }
        // The barrier orders every thread's stores before the flag writers' release, which is a
        // system-scope fence followed by the store and covers what happened before it in the CTA: one
        // fence in one warp instead of one per thread.
        __syncthreads();
        if (tid < pt.world) {
            unsigned int *f = &pt.inbox[tid]->flags[slot][pt.rank];
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(tag) : "memory");
        }
        // (the ranks' lists are merged in the idle stage buffers too when they do not fit twice into `buf`;
        //  all threads are past their reads of `buf`: the barrier above)
        CandBuf pbuf = buf;
        if (spare != nullptr && 2 * pt.world * a.k > pbuf.cap) {
            int want = pbuf.cap;
            while (want < 2 * pt.world * a.k && want * 2 <= spare_keys) want <<= 1;
            pbuf.keys = spare;
            pbuf.cap = want;
            pbuf.limit = want - kScanThreads;
        }
        if (a.defer == 0) {
            cnt = peer_merge_emit<TYPE>(pt, a.seq, a.k, pbuf, a.out_ids, a.out_scores, a.out_iscores);
        } else if (a.d_out_ids != nullptr) {
            cnt = peer_merge_emit<TYPE>(pt, a.seq - (unsigned)a.defer, a.k, pbuf, a.d_out_ids, a.d_out_scores, a.d_out_iscores);
            count_to = a.d_out_count;
        } else {
            count_to = nullptr;  // merged later, by a following launch or the drain
        }
    }
    // results may sit in host memory: all threads' writes are ordered before thread 0's system-scope
    // fence below by this barrier (one fence for the CTA, not one per thread)
    if (a.done_flag != nullptr) __syncthreads();
    if (tid == 0) {
        if (count_to != nullptr) *count_to = cnt;
        if (a.error != nullptr) *a.error = 0;
        if (a.next_batch != nullptr) *a.next_batch = 0u;
        *a.ticket = 0u;
        if (a.done_flag != nullptr) {  // (the release is the system-scope fence: none before it)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.done_flag), "r"(a.done_value) : "memory");
        }
    }
}

template <int TYPE>
__global__ void __launch_bounds__(kScanThreads, 1) k_peer_drain(const DrainArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    for (int q = 0; q < a.count; ++q) {
        const size_t o = (size_t)q * a.k;
        const int cnt = peer_merge_emit<TYPE>(*a.peer, a.seq_first + (unsigned)q, a.k, buf, a.out_ids + o, a.out_scores + o,
                                              a.out_iscores ? a.out_iscores + o : nullptr);
        if (threadIdx.x == 0) a.out_count[q] = cnt;
    }
}

// The meeting point of the free-running warps (see the header comment): returns
// true when every warp is out of rows and the buffer holds the CTA's final list.
__device__ __forceinline__ bool cand_rendezvous(const CandBuf &buf, bool work, bool &counted, int lane, int nwarps) {
    if (!work && !counted) {
        if (lane == 0) atomicAdd(&buf.ctrl->n_done, 1);
        counted = true;
    }
    __syncthreads();  // nobody appends past this point
    const int c = buf.ctrl->count, nd = buf.ctrl->n_done;
    __syncthreads();  // everybody has read the same state
    if (c > buf.limit || nd == nwarps) cand_prune(buf);
    return nd == nwarps;
}

// ---------------------------------------------------------------------------
// Scan kernel, register-staged: every lane loads its 16-byte chunks straight from
// global memory.  Used for allow-list (gathered) scans and for small inputs.
// ---------------------------------------------------------------------------
template <class TR, int TYPE, int G>
__global__ void __launch_bounds__(kScanThreads, 2) k_scan(const __grid_constant__ ScanArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int R = (G < TR::kRows) ? G : TR::kRows;

    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    unsigned char *qs = smem + (size_t)buf.cap * 8 + 16;
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < buf.cap; i += kScanThreads) buf.keys[i] = 0ull;
    if (tid == 0) {
        buf.ctrl->count = 0;
        buf.ctrl->n_done = 0;
        buf.ctrl->thr = a.floor ? __ldcg(a.floor) : 0ull;
    }
    TR::stage_query(qs, a.query != nullptr ? a.query : a.query_inline, a.chunks);
    const unsigned long long bound = a.bound ? __ldcg(a.bound) : ~0ull;
    __syncthreads();

    const long long n_batches = (a.n + 31) >> 5;
    const long long b_lo = n_batches * blockIdx.x / gridDim.x;
    const long long b_hi = n_batches * (blockIdx.x + 1) / gridDim.x;

    long long b = b_lo + warp;
    bool counted = false;
    for (;;) {
        const bool work = b < b_hi;
        int seen = 0;
        if (lane == 0) seen = *(volatile int *)&buf.ctrl->count;
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (work && seen <= buf.limit) {
            // ---- one batch: rows [32b, 32b+32) ----
            const long long row0 = b << 5;
            int myslot = 0;
            if (a.slots != nullptr && row0 + lane < a.n) myslot = a.slots[row0 + lane];
            typename TR::acc_t acc[G];
#pragma unroll
            for (int t = 0; t < G; ++t) acc[t] = (typename TR::acc_t)0;
            batch_accumulate<TR, G, R, LoadGlobal>(
                acc, qs, a.chunks, 0, a.chunks, lane,
                [&](int i) -> const unsigned char * {
                    long long srow = row0 + i;
                    if (a.slots != nullptr) srow = __shfl_sync(0xffffffffu, myslot, i);
                    return a.rows + ((row0 + i < a.n) ? srow : 0) * a.ld;
                },
                [&](int i) -> bool { return row0 + i < a.n; });
            const typename TR::acc_t total = batch_reduce<TR, G>(acc, lane);
            const long long rr = row0 + lane;
            const bool valid = rr < a.n;
            const unsigned slot = (a.slots != nullptr) ? (unsigned)myslot : (unsigned)rr;
            unsigned long long key = 0ull;
            if (valid) key = make_key(TR::finish(total, a, slot), slot);
            const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
            cand_offer_warp(buf, valid && key > thr && key < bound, key);
            b += kScanWarps;
            continue;
        }
        if (cand_rendezvous(buf, work, counted, lane, kScanWarps)) break;
    }
    publish_and_finish<TYPE>(a, buf, &s_last);
}

// ---------------------------------------------------------------------------
// Scan kernel, TMA-staged: the corpus is streamed into shared memory with bulk
// asynchronous copies (cp.async.bulk, completion on an mbarrier), 32 rows
// (32 x ld contiguous bytes) per tile.  One CTA per SM; every warp owns kStages
// private tile buffers, reads a tile with conflict-free 16-byte shared loads and,
// as soon as it has consumed it, issues the copy of its next tile into the same
// buffer.  Bytes in flight per SM = warps x (kStages-1..kStages) x tile, independent
// of register pressure, which is what it takes to keep HBM3e busy from 148 SMs.
// ---------------------------------------------------------------------------
#ifndef LK_BULK_STAGES
#define LK_BULK_STAGES 2
#endif
#ifndef LK_BULK_WARPS
#define LK_BULK_WARPS 4
#endif
constexpr int kBulkStages = LK_BULK_STAGES;
// SC > 0 fixes the slab width at compile time (SC 16-byte chunks, G must divide SC);
// SC == 0 takes it from slab_bytes.  QREG keeps the query in registers (one slab per row).

template <class TR, int TYPE, int G, int WARPS, int SC, bool QREG>
__global__ void __launch_bounds__(WARPS * 32, 1) k_scan_bulk(const __grid_constant__ ScanArgs a, int slab_bytes_rt, int n_slabs_rt) {
    const int slab_bytes = SC > 0 ? SC * 16 : slab_bytes_rt;
    const int n_slabs = QREG ? 1 : n_slabs_rt;
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int R = (G < 4) ? G : 4;  // shared-memory latency is short: few rows in flight suffice
    constexpr int T = WARPS * 32;
    using acc_t = typename TR::acc_t;

    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(smem + (size_t)buf.cap * 8 + 16);
    unsigned char *qs = smem + (size_t)buf.cap * 8 + 16 + WARPS * kBulkStages * 8;
    const size_t stage_bytes = (size_t)32 * slab_bytes;
    const size_t q_bytes = (size_t)a.chunks * TR::kQBytes;
    unsigned char *stages = smem + (((size_t)buf.cap * 8 + 16 + WARPS * kBulkStages * 8 + q_bytes + 127) & ~(size_t)127);
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Let the next launch on the stream begin as soon as SMs fall free: consecutive
    // queries are independent until they publish (see the wait before the publish).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int i = 0; i < WARPS * kBulkStages; ++i) mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();  // barriers are initialised: the first copies can go out before anything else

    const long long n_batches = (a.n + 31) >> 5;
    unsigned char *my_stages = stages + (size_t)warp * kBulkStages * stage_bytes;
    unsigned long long *my_bars = bars + warp * kBulkStages;

    // Work is handed out dynamically: a warp takes the next 32-row batch from a global
    // counter whenever one of its stages falls free, so SMs that get more bandwidth
    // simply take more batches and all SMs finish together.  A batch is loaded in
    // n_slabs items (column ranges of slab_bytes of each row; the last may be narrower;
    // rows sit slab-width bytes apart in the stage); item m of a warp lives in stage
    // m % kBulkStages and items are consumed in the order they were issued.
    auto slab_width = [&](int sl) -> int { return min(slab_bytes, (int)a.ld - sl * slab_bytes); };
    long long stage_batch[kBulkStages];  // batch held by each stage, -1 = none
#pragma unroll
    for (int s = 0; s < kBulkStages; ++s) stage_batch[s] = -1;
    long long iss_batch = -1;  // batch whose slabs are being issued
    int iss_slab = 0;
    bool exhausted = false;
    // The first kBulkStages batches of every warp are fixed (no round trip to the
    // counter before the first copy); the counter hands out the batches after those.
    const long long static_base = ((long long)blockIdx.x * WARPS + warp) * kBulkStages;
    const long long first_dynamic = (long long)gridDim.x * WARPS * kBulkStages;
    int static_used = 0;
    auto issue = [&](int s) {  // called by the whole warp: fill stage s with the next item
        long long bnew = -1;
        if (iss_slab == 0) {
            if (!exhausted) {
                long long t;
                if (static_used < kBulkStages) {
                    t = static_base + static_used++;
                } else {
                    unsigned d = 0;
                    if (lane == 0) d = atomicAdd(a.next_batch, 1u);
                    t = first_dynamic + (long long)__shfl_sync(0xffffffffu, d, 0);
                }
                if (t < n_batches) iss_batch = t; else exhausted = true;
            }
            if (exhausted) iss_batch = -1;
        }
        bnew = iss_batch;
#pragma unroll
        for (int i = 0; i < kBulkStages; ++i)
            if (i == s) stage_batch[i] = bnew;
        if (bnew < 0) return;
        const int sl = iss_slab;
        iss_slab = (iss_slab + 1 == n_slabs) ? 0 : iss_slab + 1;
        const long long row0 = bnew << 5;
        const int rows = (int)min(32ll, a.n - row0);
        const int w = slab_width(sl);
        unsigned char *dst = my_stages + (size_t)s * stage_bytes;
        if (lane == 0) mbar_expect_tx(&my_bars[s], (unsigned)(rows * w));
        __syncwarp();
        if (n_slabs == 1) {  // whole rows: the batch is one contiguous range
            if (lane == 0) bulk_load(dst, a.rows + (size_t)row0 * a.ld, (unsigned)(rows * w), &my_bars[s]);
        } else if (lane < rows) {  // one row segment per lane
            bulk_load(dst + (size_t)lane * w, a.rows + (size_t)(row0 + lane) * a.ld + (size_t)sl * slab_bytes,
                      (unsigned)w, &my_bars[s]);
        }
    };
#pragma unroll
    for (int s = 0; s < kBulkStages; ++s) issue(s);

    // the rest of the prologue runs while the first copies are in flight
    for (int i = tid; i < buf.cap; i += T) buf.keys[i] = 0ull;
    if (tid == 0) {
        buf.ctrl->count = 0;
        buf.ctrl->n_done = 0;
        buf.ctrl->thr = 0ull;
    }
    TR::stage_query(qs, a.query != nullptr ? a.query : a.query_inline, a.chunks);
    unsigned long long bound = ~0ull;
    if (a.bound != nullptr || a.floor != nullptr) {
        // a later pass of a large-k search (its bound is the previous pass's output) or a search with a
        // sampled floor that the launch just before has written: wait for that launch
        if (a.bound != nullptr || a.floor_wait != 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (a.bound != nullptr) bound = __ldcg(a.bound);
        if (a.floor != nullptr && tid == 0) buf.ctrl->thr = __ldcg(a.floor);
    }
    __syncthreads();

    constexpr int NJ = SC > 0 ? SC / G : 1;
    typename TR::QChunk qreg[NJ];
    if (QREG) {
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) qreg[jj] = TR::load_q(qs, (lane % G) + jj * G, a.chunks);
    }

    long long m = 0;
    bool counted = false, failed = false;
    // small k without a bound: the warp keeps its best keys in registers (warp_top_offer)
    const bool regk = a.k <= 32 && a.bound == nullptr && a.floor == nullptr;
    unsigned long long wk = 0ull, wthr = 0ull;
    acc_t acc[G];
    for (;;) {
        const int s = (int)(m % kBulkStages);
        const int sl = (int)(m % n_slabs);
        long long b = -1;
#pragma unroll
        for (int i = 0; i < kBulkStages; ++i)
            if (i == s) b = stage_batch[i];
        const bool work = b >= 0 && !failed;
        int seen = 0;
        if (lane == 0) seen = *(volatile int *)&buf.ctrl->count;
        seen = __shfl_sync(0xffffffffu, seen, 0);
        // the buffer is only looked at between batches: a batch in progress always finishes
        if (work && (sl != 0 || seen <= buf.limit)) {
            const unsigned parity = (unsigned)((m / kBulkStages) & 1);
            // bounded wait for the data; on expiry flag the error and stop taking work
            unsigned spins = 0;
            bool ready = false;
            while (!(ready = mbar_try_wait(&my_bars[s], parity)) && ++spins < kBulkSpinLimit) {}
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0 && a.error != nullptr) atomicExch(a.error, 1);
                failed = true;
                continue;
            }
            const long long row0 = b << 5;
            const int rows = (int)min(32ll, a.n - row0);
            const int w = slab_width(sl);
            const unsigned char *stage = my_stages + (size_t)s * stage_bytes;
            if (sl == 0) {
#pragma unroll
                for (int t = 0; t < G; ++t) acc[t] = (acc_t)0;
            }
            // Rows past the end of a short last batch hold stale bytes: they are scored like any
            // other (shared memory is always readable) and dropped by `valid` below.
            if (SC > 0) {
                if (QREG) {
                    slab_accumulate_fixed<TR, G, (SC > 0 ? SC : G)>(acc, qreg, stage, lane);
                } else {
                    typename TR::QChunk q[NJ];
#pragma unroll
                    for (int jj = 0; jj < NJ; ++jj) q[jj] = TR::load_q(qs, sl * SC + (lane % G) + jj * G, a.chunks);
                    slab_accumulate_fixed<TR, G, (SC > 0 ? SC : G)>(acc, q, stage, lane);
                }
            } else {
                batch_accumulate<TR, G, R, LoadShared>(
                    acc, qs, a.chunks, sl * (slab_bytes >> 4), w >> 4, lane,
                    [&](int i) -> const unsigned char * { return stage + (size_t)i * w; },
                    [&](int) -> bool { return true; });
            }
            // every lane has its part of the stage in registers (the accumulators depend on
            // it): the stage is free, refill it with this warp's next item
            __syncwarp();
            issue(s);
            ++m;
            if (sl != n_slabs - 1) continue;
            const acc_t total = batch_reduce<TR, G>(acc, lane);
            const bool valid = lane < rows;
            const unsigned slot = (unsigned)(row0 + lane);
            unsigned long long key = 0ull;
            if (valid) key = make_key(TR::finish(total, a, slot), slot);
            if (regk) {
                warp_top_offer(wk, wthr, a.k, valid && key > wthr, key, lane);
            } else {
                const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
                cand_offer_warp(buf, valid && key > thr && key < bound, key);
            }
            continue;
        }
        if (regk && !work && !counted) cand_offer_warp(buf, lane < a.k && wk != 0ull, wk);  // hand the warp's list over, once
        if (cand_rendezvous(buf, work, counted, lane, WARPS)) break;
    }
    // A warp that gave up may still have copies in flight into its stages: wait for
    // them (bounded) before the CTA's shared memory is released.
    if (failed) {
        for (long long mm = m; mm < m + kBulkStages; ++mm) {
            long long b = -1;
#pragma unroll
            for (int i = 0; i < kBulkStages; ++i)
                if (i == (int)(mm % kBulkStages)) b = stage_batch[i];
            if (b < 0) continue;
            unsigned spins = 0;
            while (!mbar_try_wait(&my_bars[mm % kBulkStages], (unsigned)((mm / kBulkStages) & 1)) &&
                   ++spins < kBulkSpinLimit) {}
        }
    }
    // Everything up to here touched only this launch's own state.  The scratch shared
    // with the previous launch on the stream (per-CTA lists, ticket) is next: wait until
    // that launch has completely finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();  // every warp is done with its stages: they are the last CTA's merge space
    publish_and_finish<TYPE>(a, buf, &s_last, reinterpret_cast<unsigned long long *>(stages),
                             (int)((size_t)WARPS * kBulkStages * stage_bytes / 8));
}

// ---------------------------------------------------------------------------
// TMA-staged scan for WIDE rows (ld a multiple of 512 bytes, 1 KB and up).
// A batch is RB whole rows = one contiguous bulk copy of RB * ld bytes.  All 32
// lanes share a row: lane l reads 16-byte chunks l, l+32, ... (NJ of them), keeps
// one accumulator per row of the batch and the query chunks it needs in registers.
// Float rows pay one float32->float64 conversion per element on a 16-lane-per-clock
// pipe, whose latency a single warp per scheduler cannot hide: the float kernels
// run 8 warps per CTA with half-size stages, the int8 kernel 4.
// Batches are handed out in runs of `run` consecutive batches per counter access.
// ---------------------------------------------------------------------------
template <class TR, int RB>
__device__ __forceinline__ typename TR::acc_t wide_reduce(typename TR::acc_t (&acc)[RB], int lane) {
    using acc_t = typename TR::acc_t;
    // plain halving down to RB lanes per value, then the transposed butterfly
#pragma unroll
    for (int w = 16; w >= RB; w >>= 1) {
#pragma unroll
        for (int i = 0; i < RB; ++i) acc[i] = acc[i] + TR::shfl(acc[i], w);
    }
#pragma unroll
    for (int w = RB / 2; w >= 1; w >>= 1) {
        const bool upper = (lane & w) != 0;
#pragma unroll
        for (int i = 0; i < w; ++i) {
            const acc_t send = upper ? acc[i] : acc[i + w];
            const acc_t keep = upper ? acc[i + w] : acc[i];
            acc[i] = keep + TR::shfl(send, w);
        }
    }
    return acc[0];  // lane i (mod RB) holds row i
}

template <class TR, int TYPE, int WARPS, int RB, int NJ>
__global__ void __launch_bounds__(WARPS * 32, 1) k_scan_wide(const __grid_constant__ ScanArgs a, int run) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int T = WARPS * 32;
    constexpr int LD = NJ * 512;
    constexpr int STAGE = RB * LD;
    using acc_t = typename TR::acc_t;

    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(smem + (size_t)buf.cap * 8 + 16);
    unsigned char *qs = smem + (size_t)buf.cap * 8 + 16 + WARPS * kBulkStages * 8;
    const size_t q_bytes = (size_t)a.chunks * TR::kQBytes;
    unsigned char *stages = smem + (((size_t)buf.cap * 8 + 16 + WARPS * kBulkStages * 8 + q_bytes + 127) & ~(size_t)127);
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int i = 0; i < WARPS * kBulkStages; ++i) mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const long long n_batches = (a.n + RB - 1) / RB;
    unsigned char *my_stages = stages + (size_t)warp * kBulkStages * STAGE;
    unsigned long long *my_bars = bars + warp * kBulkStages;

    // batch hand-out: the first run of every warp is fixed, later runs come from the counter
    const long long static_run = (long long)blockIdx.x * WARPS + warp;
    const long long first_dynamic = (long long)gridDim.x * WARPS;
    long long run_next = 0, run_end = 0;  // batches [run_next, run_end) of the current run
    bool first = true, exhausted = false;
    long long stage_batch[kBulkStages];
#pragma unroll
    for (int s = 0; s < kBulkStages; ++s) stage_batch[s] = -1;
    auto issue = [&](int s) {  // whole warp
        if (run_next >= run_end && !exhausted) {
            long long r;
            if (first) {
                r = static_run;
                first = false;
            } else {
                unsigned d = 0;
                if (lane == 0) d = atomicAdd(a.next_batch, 1u);
                r = first_dynamic + (long long)__shfl_sync(0xffffffffu, d, 0);
            }
            run_next = r * run;
            run_end = min(run_next + run, n_batches);
            if (run_next >= n_batches) exhausted = true;
        }
        const long long b = (!exhausted && run_next < run_end) ? run_next++ : -1;
#pragma unroll
        for (int i = 0; i < kBulkStages; ++i)
            if (i == s) stage_batch[i] = b;
        if (b < 0) return;
        if (lane == 0) {
            const long long row0 = b * RB;
            const unsigned bytes = (unsigned)(min((long long)RB, a.n - row0) * LD);
            mbar_expect_tx(&my_bars[s], bytes);
            bulk_load(my_stages + (size_t)s * STAGE, a.rows + (size_t)row0 * LD, bytes, &my_bars[s]);
        }
    };
#pragma unroll
    for (int s = 0; s < kBulkStages; ++s) issue(s);

    for (int i = tid; i < buf.cap; i += T) buf.keys[i] = 0ull;
    if (tid == 0) {
        buf.ctrl->count = 0;
        buf.ctrl->n_done = 0;
        buf.ctrl->thr = 0ull;
    }
    TR::stage_query(qs, a.query != nullptr ? a.query : a.query_inline, a.chunks);
    unsigned long long bound = ~0ull;
    if (a.bound != nullptr || a.floor != nullptr) {
        if (a.bound != nullptr || a.floor_wait != 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (a.bound != nullptr) bound = __ldcg(a.bound);
        if (a.floor != nullptr && tid == 0) buf.ctrl->thr = __ldcg(a.floor);
    }
    __syncthreads();
    typename TR::QChunk q[NJ];
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) q[jj] = TR::load_q(qs, lane + jj * 32, a.chunks);

    long long m = 0;
    bool counted = false, failed = false;
    // small k without a bound: the warp keeps its best keys in registers (warp_top_offer)
    const bool regk = a.k <= 32 && a.bound == nullptr && a.floor == nullptr;
    unsigned long long wk = 0ull, wthr = 0ull;
    for (;;) {
        const int s = (int)(m % kBulkStages);
        long long b = -1;
#pragma unroll
        for (int i = 0; i < kBulkStages; ++i)
            if (i == s) b = stage_batch[i];
        const bool work = b >= 0 && !failed;
        int seen = 0;
        if (lane == 0) seen = *(volatile int *)&buf.ctrl->count;
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (work && seen <= buf.limit) {
            const unsigned parity = (unsigned)((m / kBulkStages) & 1);
            unsigned spins = 0;
            bool ready = false;
            while (!(ready = mbar_try_wait(&my_bars[s], parity)) && ++spins < kBulkSpinLimit) {}
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0 && a.error != nullptr) atomicExch(a.error, 1);
                failed = true;
                continue;
            }
            const unsigned char *base = my_stages + (size_t)s * STAGE + (size_t)lane * 16;
            acc_t acc[RB];
#pragma unroll
            for (int r = 0; r < RB; ++r) acc[r] = (acc_t)0;
            // rows past the end of a short last batch hold stale bytes and are dropped by `valid`
#pragma unroll
            for (int r = 0; r < RB; ++r) {
#pragma unroll
                for (int jj = 0; jj < NJ; ++jj) {
                    const int4 v = *reinterpret_cast<const int4 *>(base + r * LD + jj * 512);
                    TR::dot(acc[r], v, q[jj]);
                }
            }
            __syncwarp();  // all lanes have the stage in registers: refill it
            issue(s);
            ++m;
            const acc_t total = wide_reduce<TR, RB>(acc, lane);
            const long long row = b * RB + (lane % RB);
            const bool valid = lane < RB && row < a.n;
            const unsigned slot = (unsigned)row;
            unsigned long long key = 0ull;
            if (valid) key = make_key(TR::finish(total, a, slot), slot);
            if (regk) {
                warp_top_offer(wk, wthr, a.k, valid && key > wthr, key, lane);
            } else {
                const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
                cand_offer_warp(buf, valid && key > thr && key < bound, key);
            }
            continue;
        }
        if (regk && !work && !counted) cand_offer_warp(buf, lane < a.k && wk != 0ull, wk);  // hand the warp's list over, once
        if (cand_rendezvous(buf, work, counted, lane, WARPS)) break;
    }
    if (failed) {
        for (long long mm = m; mm < m + kBulkStages; ++mm) {
            long long b = -1;
#pragma unroll
            for (int i = 0; i < kBulkStages; ++i)
                if (i == (int)(mm % kBulkStages)) b = stage_batch[i];
            if (b < 0) continue;
            unsigned spins = 0;
            while (!mbar_try_wait(&my_bars[mm % kBulkStages], (unsigned)((mm / kBulkStages) & 1)) &&
                   ++spins < kBulkSpinLimit) {}
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();  // every warp is done with its stages: they are the last CTA's merge space
    publish_and_finish<TYPE>(a, buf, &s_last, reinterpret_cast<unsigned long long *>(stages),
                             (int)((size_t)WARPS * kBulkStages * STAGE / 8));
}

// ---------------------------------------------------------------------------
// Brute-force scan over RAW rows with the reference's CosineSim
// (media-server/embedvec/embedvec.go:127-141): float32(dot / (sqrt(|q|^2) * sqrt(|v|^2))),
// everything accumulated in float64, 0 when either vector is all zero.  This is the scoring
// of the service layer's fallbacks, which run over the un-normalised vectors as the database
// holds them (media-server/tasks/embed_task.go:249-272, media-server/tasks/face_search.go:199-216,
// :235-248).  a.rows holds n_rows x dim floats, dim * 4 bytes apart (no padding, any alignment
// of 4); a.query dim floats.  A warp takes 32 rows at a time, four rows in flight, all lanes on
// one row; top-k and the final merge are the scan's.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kScanThreads, 2) k_cosine_sim(const __grid_constant__ ScanArgs a, int dim, double q_n2) {
    extern __shared__ __align__(128) unsigned char smem[];
    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    double *qs = reinterpret_cast<double *>(smem + (size_t)buf.cap * 8 + 16);
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < buf.cap; i += kScanThreads) buf.keys[i] = 0ull;
    if (tid == 0) {
        buf.ctrl->count = 0;
        buf.ctrl->n_done = 0;
        buf.ctrl->thr = 0ull;
    }
    const float *qf = reinterpret_cast<const float *>(a.query);
    for (int j = tid; j < dim; j += kScanThreads) qs[j] = (double)qf[j];
    const unsigned long long bound = a.bound ? __ldcg(a.bound) : ~0ull;  // later pass of a large-k search
    __syncthreads();
    const float *rows = reinterpret_cast<const float *>(a.rows);
    const double q_norm = sqrt(q_n2);
    const long long n_batches = (a.n + 31) >> 5;
    const long long b_lo = n_batches * blockIdx.x / gridDim.x;
    const long long b_hi = n_batches * (blockIdx.x + 1) / gridDim.x;
    long long b = b_lo + warp;
    bool counted = false;
    for (;;) {
        const bool work = b < b_hi;
        int seen = 0;
        if (lane == 0) seen = *(volatile int *)&buf.ctrl->count;
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (work && seen <= buf.limit) {
            const long long row0 = b << 5;
            int myslot = 0;
            if (row0 + lane < a.n) myslot = a.slots ? a.slots[row0 + lane] : (int)(row0 + lane);
            double my_dot = 0.0, my_n2 = 0.0;
            for (int r0 = 0; r0 < 32; r0 += 4) {
                const float *p[4];
                double dot[4] = {0.0, 0.0, 0.0, 0.0}, n2[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int s = __shfl_sync(0xffffffffu, myslot, r0 + r);
                    p[r] = rows + (size_t)s * dim;  // rows past the end alias row 0 and are dropped below
                }
                for (int j = lane; j < dim; j += 32) {
                    const double q = qs[j];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const double v = (double)__ldg(p[r] + j);
                        dot[r] = fma(v, q, dot[r]);   // float32 products are exact in float64
                        n2[r] = fma(v, v, n2[r]);
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
#pragma unroll
                    for (int w = 16; w >= 1; w >>= 1) {
                        dot[r] += TraitsF32::shfl(dot[r], w);
                        n2[r] += TraitsF32::shfl(n2[r], w);
                    }
                    if (lane == r0 + r) {
                        my_dot = dot[r];
                        my_n2 = n2[r];
                    }
                }
            }
            const bool valid = row0 + lane < a.n;
            float score = 0.0f;
            if (q_n2 != 0.0 && my_n2 != 0.0) score = (float)(my_dot / (q_norm * sqrt(my_n2)));
            unsigned long long key = 0ull;
            if (valid) key = make_key(ord_from_f32(score), (unsigned)myslot);
            const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
            cand_offer_warp(buf, valid && key > thr && key < bound, key);
            b += kScanWarps;
            continue;
        }
        if (cand_rendezvous(buf, work, counted, lane, kScanWarps)) break;
    }
    publish_and_finish<SCAN_F32>(a, buf, &s_last);
}

int cosine_sim_launch(const ScanArgs &a, int dim, double q_n2, int sm_count, cudaStream_t stream, int *grid_out) {
    const size_t smem = (size_t)cand_capacity(a.k) * 8 + 16 + (size_t)dim * 8;
    cudaError_t e = cudaFuncSetAttribute((const void *)k_cosine_sim, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(4, std::string("cosine_sim attr: ") + cudaGetErrorString(e));
    const long long batches = (a.n + 31) / 32;
    const int grid = (int)std::max<long long>(1, std::min<long long>(batches, (long long)sm_count * 2));
    if (grid_out) *grid_out = grid;
    if (a.part == nullptr) return 0;  // sizing call
    k_cosine_sim<<<grid, kScanThreads, smem, stream>>>(a, dim, q_n2);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("cosine_sim launch: ") + cudaGetErrorString(e));
    return 0;
}

// ---------------------------------------------------------------------------
// Merge of ranked lists (after the all-gather of per-shard candidates)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kScanThreads, 1) k_merge_lists(const MergeArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    const int tid = threadIdx.x;
    const int q = blockIdx.x;
    const long long total = (long long)a.lists * a.k;
    unsigned long long *scratch = a.scratch + (size_t)q * total;
    long long *out_ids = a.out_ids + (size_t)q * a.k;
    float *out_scores = a.out_scores + (size_t)q * a.k;
    int *out_iscores = a.out_iscores ? a.out_iscores + (size_t)q * a.k : nullptr;
    // list l of this query starts at keys[(l*nq + q)*k]
    // Re-base every key to global ids: the low word holds ~id, so subtracting the
    // list's base from the key adds it to the id.
    for (long long i = tid; i < total; i += kScanThreads) {
        const int l = (int)(i / a.k), j = (int)(i % a.k);
        unsigned long long key = a.keys[((size_t)l * a.nq + q) * a.k + j];
        if (key != 0ull) key -= (unsigned long long)a.list_base[l];
        scratch[i] = key;
    }
    __threadfence_block();
    __syncthreads();
    cand_select_from_lists(buf, scratch, a.lists);
    const int cnt = buf.ctrl->count;
    for (int i = tid; i < a.k; i += kScanThreads) {
        const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
        if (a.out_keys) a.out_keys[(size_t)q * a.k + i] = key;
        if (key == 0ull) {
            out_ids[i] = -1;
            out_scores[i] = 0.0f;
            if (out_iscores) out_iscores[i] = 0;
            continue;
        }
        const long long gid = (long long)key_slot(key);
        out_ids[i] = gid;
        if (a.type != SCAN_I8) {
            out_scores[i] = f32_from_ord(key_ord(key));
            if (out_iscores) out_iscores[i] = 0;
            continue;
        }
        if (a.payload == nullptr) {  // single GPU: the row scales are here
            const int isc = i32_from_ord(key_ord(key));
            out_scores[i] = (float)isc * (a.qscales[q] * a.scales[gid]);
            if (out_iscores) out_iscores[i] = isc;
            continue;
        }
        // int8: the float score was finished by the shard that owns the row (it needs
        // the row's scale); find the key in its origin list (ranked descending).
        int l = 0;
        for (int t = 1; t < a.lists; ++t)
            if (a.list_base[t] <= gid) l = t;
        const unsigned long long orig = key + (unsigned long long)a.list_base[l];
        const size_t lo0 = ((size_t)l * a.nq + q) * a.k;
        int lo = 0, hi = a.k - 1;
        float sc = 0.0f;
        while (lo <= hi) {
            const int mid = (lo + hi) >> 1;
            const unsigned long long v = a.keys[lo0 + mid];
            if (v == orig) { sc = a.payload[lo0 + mid]; break; }
            if (v > orig) lo = mid + 1; else hi = mid - 1;
        }
        out_scores[i] = sc;
        if (out_iscores) out_iscores[i] = i32_from_ord(key_ord(key));
    }
    if (tid == 0) a.out_count[q] = cnt;
}

// ---------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------
int scan_group_width(int chunks) {
    int best = 32, best_waste = 1 << 30;
    for (int g = 32; g >= 1; g >>= 1) {
        const int padded = (chunks + g - 1) / g * g;
        const int waste = padded - chunks;
        if (waste < best_waste) {
            best_waste = waste;
            best = g;
        }
    }
    return best;
}

int scan_query_bytes(int type, long long ld) {
    switch (type) {
        case SCAN_I8: return (int)ld;          // int8 codes
        case SCAN_F32: return (int)ld;         // float32, ld/4 elements
        default: return (int)(ld * 2);         // float32 query for ld/2 halves
    }
}

static int q_smem_per_chunk(int type) {
    return (type == SCAN_I8) ? TraitsI8::kQBytes : (type == SCAN_F32 ? TraitsF32::kQBytes : TraitsF16::kQBytes);
}

constexpr int kBulkWarps = LK_BULK_WARPS;
constexpr int kBulkSlabMax = 768;               // bytes of one row kept per stage: 32 rows x 768 B = 24 KB
constexpr size_t kSmemLimit = 227 * 1024;

typedef void (*scan_fn)(const ScanArgs);
typedef void (*bulk_fn)(const ScanArgs, int, int);

// slab shapes with a compile-time kernel: 48 chunks (768 B) and 32 chunks (512 B)
static int bulk_fixed_chunks(int ld) { return (ld % 768 == 0) ? 48 : ((ld % 512 == 0) ? 32 : 0); }

template <class TR, int TYPE>
static scan_fn pick_g(int g) {
    switch (g) {
        case 1: return k_scan<TR, TYPE, 1>;
        case 2: return k_scan<TR, TYPE, 2>;
        case 4: return k_scan<TR, TYPE, 4>;
        case 8: return k_scan<TR, TYPE, 8>;
        case 16: return k_scan<TR, TYPE, 16>;
        default: return k_scan<TR, TYPE, 32>;
    }
}
static scan_fn pick(int type, int g) {
    switch (type) {
        case SCAN_I8: return pick_g<TraitsI8, SCAN_I8>(g);
        case SCAN_F32: return pick_g<TraitsF32, SCAN_F32>(g);
        default: return pick_g<TraitsF16, SCAN_F16>(g);
    }
}
template <class TR, int TYPE>
static bulk_fn pick_bulk_g(int g, int sc, bool qreg) {
    if (sc == 48) return qreg ? k_scan_bulk<TR, TYPE, 16, kBulkWarps, 48, true> : k_scan_bulk<TR, TYPE, 16, kBulkWarps, 48, false>;
    if (sc == 32) return qreg ? k_scan_bulk<TR, TYPE, 32, kBulkWarps, 32, true> : k_scan_bulk<TR, TYPE, 32, kBulkWarps, 32, false>;
    switch (g) {
        case 1: return k_scan_bulk<TR, TYPE, 1, kBulkWarps, 0, false>;
        case 2: return k_scan_bulk<TR, TYPE, 2, kBulkWarps, 0, false>;
        case 4: return k_scan_bulk<TR, TYPE, 4, kBulkWarps, 0, false>;
        case 8: return k_scan_bulk<TR, TYPE, 8, kBulkWarps, 0, false>;
        case 16: return k_scan_bulk<TR, TYPE, 16, kBulkWarps, 0, false>;
        default: return k_scan_bulk<TR, TYPE, 32, kBulkWarps, 0, false>;
    }
}
static bulk_fn pick_bulk(int type, const ScanPlan &p) {
    const bool qreg = p.fixed_chunks > 0 && p.n_slabs == 1;
    switch (type) {
        case SCAN_I8: return pick_bulk_g<TraitsI8, SCAN_I8>(p.bulk_g, p.fixed_chunks, qreg);
        case SCAN_F32: return pick_bulk_g<TraitsF32, SCAN_F32>(p.bulk_g, p.fixed_chunks, qreg);
        default: return pick_bulk_g<TraitsF16, SCAN_F16>(p.bulk_g, p.fixed_chunks, qreg);
    }
}

typedef void (*wide_fn)(const ScanArgs, int);

constexpr int kWideWarpsInt = 4, kWideWarpsFloat = 8;

// (rows per batch, 512-byte units per row) -> kernel, for the widths that have one
template <class TR, int TYPE, int WARPS, int RB>
static wide_fn pick_wide_nj(int nj) {
    switch (nj) {
        case 2: return k_scan_wide<TR, TYPE, WARPS, (RB * 2 > 32 ? 32 : RB * 2), 2>;
        case 3: return k_scan_wide<TR, TYPE, WARPS, (RB * 2 > 32 ? 32 : RB * 2), 3>;
        case 4: return k_scan_wide<TR, TYPE, WARPS, RB, 4>;
        case 6: return k_scan_wide<TR, TYPE, WARPS, RB, 6>;
        case 8: return k_scan_wide<TR, TYPE, WARPS, RB / 2, 8>;
        default: return nullptr;
    }
}
static int wide_rows(int type, int nj) {  // must mirror pick_wide_nj
    const int rb = (type == SCAN_I8) ? 8 : 4;
    return nj <= 3 ? rb * 2 : (nj == 8 ? rb / 2 : rb);
}
static wide_fn pick_wide(int type, int nj) {
    switch (type) {
        case SCAN_I8: return pick_wide_nj<TraitsI8, SCAN_I8, kWideWarpsInt, 8>(nj);
        case SCAN_F32: return pick_wide_nj<TraitsF32, SCAN_F32, kWideWarpsFloat, 4>(nj);
        default: return pick_wide_nj<TraitsF16, SCAN_F16, kWideWarpsFloat, 4>(nj);
    }
}

// The dynamic shared-memory limit of a kernel is process-wide state and plans for several k coexist
// (a sample scan with a small k beside the scan proper): the limit is always raised to the most a CTA
// of that kernel may have, never to what one plan needs.
static cudaError_t raise_smem_limit(const void *fn, int device) {
    int optin = 0;
    cudaError_t e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (e != cudaSuccess) return e;
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, fn);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - (int)fa.sharedSizeBytes);
}

int scan_plan(int type, int chunks, int k, int device, ScanPlan *plan) {
    ScanPlan p;
    int sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return fail(4, std::string("scan plan: ") + cudaGetErrorString(e));
    const size_t head = (size_t)cand_capacity(k) * 8 + 16;
    const size_t q = (size_t)chunks * q_smem_per_chunk(type);
    // register-staged kernel
    p.g = scan_group_width(chunks);
    p.smem = head + q;
    {
        scan_fn fn = pick(type, p.g);
        e = raise_smem_limit((const void *)fn, device);
        int per_sm = 0;
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void *)fn, kScanThreads, p.smem);
        if (e != cudaSuccess) return fail(4, std::string("scan plan: ") + cudaGetErrorString(e));
        p.grid = std::max(per_sm, 1) * sms;
    }
    // TMA-staged kernel
    const int ld = chunks * 16;
    p.fixed_chunks = bulk_fixed_chunks(ld);
    if (p.fixed_chunks > 0) {
        p.slab_bytes = p.fixed_chunks * 16;
        p.n_slabs = ld / p.slab_bytes;
    } else {
        p.n_slabs = (ld + kBulkSlabMax - 1) / kBulkSlabMax;
        p.slab_bytes = (int)round_up((ld + p.n_slabs - 1) / p.n_slabs, 16);
    }
    p.bulk_g = scan_group_width(p.slab_bytes / 16);
    p.bulk_smem = ((head + kBulkWarps * kBulkStages * 8 + q + 127) & ~(size_t)127) +
                  (size_t)kBulkWarps * kBulkStages * 32 * p.slab_bytes;
    p.bulk_ok = p.bulk_smem <= kSmemLimit;
    p.bulk_grid = sms;
    // wide rows: whole-row batches (k_scan_wide)
    p.wide_nj = (ld >= 1024 && ld % 512 == 0) ? ld / 512 : 0;
    if (p.wide_nj > 0 && pick_wide(type, p.wide_nj) != nullptr) {
        p.wide_warps = (type == SCAN_I8) ? kWideWarpsInt : kWideWarpsFloat;
        p.wide_rows = wide_rows(type, p.wide_nj);
        const size_t stage = (size_t)p.wide_rows * ld;
        p.wide_smem = ((head + p.wide_warps * kBulkStages * 8 + q + 127) & ~(size_t)127) +
                      (size_t)p.wide_warps * kBulkStages * stage;
        p.wide_run = (int)std::max<size_t>(1, (size_t)24576 / stage);
        if (p.wide_smem <= kSmemLimit) {
            e = raise_smem_limit((const void *)pick_wide(type, p.wide_nj), device);
            if (e != cudaSuccess) return fail(4, std::string("scan plan (wide): ") + cudaGetErrorString(e));
            p.wide_ok = true;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&p.wide_per_sm, (const void *)pick_wide(type, p.wide_nj),
                                                              p.wide_warps * 32, p.wide_smem);
            if (e != cudaSuccess) return fail(4, std::string("scan plan (wide): ") + cudaGetErrorString(e));
        }
    }
    if (p.bulk_ok) {
        bulk_fn fn = pick_bulk(type, p);
        e = raise_smem_limit((const void *)fn, device);
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&p.bulk_per_sm, (const void *)fn, kBulkWarps * 32, p.bulk_smem);
        if (e != cudaSuccess) return fail(4, std::string("scan plan (bulk): ") + cudaGetErrorString(e));
    }
    *plan = p;
    return 0;
}

bool scan_may_overlap(const ScanPlan &plan, long long launch_index) {
    const bool several_per_sm = (plan.bulk_ok && plan.bulk_per_sm > 1) || (plan.wide_ok && plan.wide_per_sm > 1);
    return !(several_per_sm && launch_index % kScanOverlap == 0);
}

int scan_launch(int type, const ScanArgs &a, const ScanPlan &plan, cudaStream_t stream, bool overlap) {
    const long long batches = (a.n + 31) / 32;
    // the TMA-staged kernel needs whole, contiguous rows and enough batches to fill its pipeline
    const bool bulk = plan.bulk_ok && a.slots == nullptr && batches >= (long long)plan.bulk_grid * kBulkWarps;
    const bool wide = plan.wide_ok && a.slots == nullptr &&
                      a.n >= (long long)plan.bulk_grid * plan.wide_warps * plan.wide_rows * plan.wide_run * 2;
    if (wide) {
        wide_fn fn = pick_wide(type, plan.wide_nj);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)plan.bulk_grid);
        cfg.blockDim = dim3(plan.wide_warps * 32);
        cfg.dynamicSmemBytes = plan.wide_smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap ? 1 : 0;
        cudaError_t le = cudaLaunchKernelEx(&cfg, fn, a, plan.wide_run);
        if (le != cudaSuccess) return fail(4, std::string("scan launch: ") + cudaGetErrorString(le));
    } else if (bulk) {
        bulk_fn fn = pick_bulk(type, plan);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)plan.bulk_grid);
        cfg.blockDim = dim3(kBulkWarps * 32);
        cfg.dynamicSmemBytes = plan.bulk_smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap ? 1 : 0;
        cudaError_t le = cudaLaunchKernelEx(&cfg, fn, a, plan.slab_bytes, plan.n_slabs);
        if (le != cudaSuccess) return fail(4, std::string("scan launch: ") + cudaGetErrorString(le));
    } else {
        scan_fn fn = pick(type, plan.g);
        // never more CTAs than give every warp of a CTA a batch: fewer lists for the last CTA to merge
        int grid = plan.grid;
        const long long full = batches / kScanWarps;
        if (full < grid) grid = (int)(full > 0 ? full : 1);
        fn<<<grid, kScanThreads, plan.smem, stream>>>(a);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("scan launch: ") + cudaGetErrorString(e));
    return 0;
}

int peer_drain_launch(const DrainArgs &a, cudaStream_t stream) {
    const size_t smem = (size_t)cand_capacity(a.k) * 8 + 16;
    void (*fn)(const DrainArgs) = a.type == SCAN_I8 ? k_peer_drain<SCAN_I8> : (a.type == SCAN_F32 ? k_peer_drain<SCAN_F32> : k_peer_drain<SCAN_F16>);
    fn<<<1, kScanThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("drain launch: ") + cudaGetErrorString(e));
    return 0;
}

int scan_max_grid(const ScanPlan &plan) { return std::max(plan.grid, plan.bulk_grid); }

int merge_launch(const MergeArgs &a, cudaStream_t stream) {
    const size_t smem = (size_t)cand_capacity(a.k) * 8 + 16;
    cudaError_t e = cudaFuncSetAttribute((const void *)k_merge_lists, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(4, std::string("merge attr: ") + cudaGetErrorString(e));
    k_merge_lists<<<a.nq, kScanThreads, smem, stream>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("merge launch: ") + cudaGetErrorString(e));
    return 0;
}

}  // namespace lk
