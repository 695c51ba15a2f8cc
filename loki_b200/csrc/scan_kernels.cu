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
    __device__ __forceinline__ static void dot(acc_t &acc, const int4 &v, const QChunk &c) {
        acc = fma((double)__int_as_float(v.x), c.a.x, acc);
        acc = fma((double)__int_as_float(v.y), c.a.y, acc);
        acc = fma((double)__int_as_float(v.z), c.b.x, acc);
        acc = fma((double)__int_as_float(v.w), c.b.y, acc);
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
// The scan kernel
// ---------------------------------------------------------------------------
template <class TR, int TYPE, int G>
__global__ void __launch_bounds__(kScanThreads, 2) k_scan(const ScanArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int R = (G < TR::kRows) ? G : TR::kRows;
    using acc_t = typename TR::acc_t;

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
        buf.ctrl->thr = 0ull;
    }
    TR::stage_query(qs, a.query, a.chunks);
    const unsigned long long bound = a.bound ? __ldcg(a.bound) : ~0ull;
    __syncthreads();

    const long long n_batches = (a.n + 31) >> 5;
    const long long b_lo = n_batches * blockIdx.x / gridDim.x;
    const long long b_hi = n_batches * (blockIdx.x + 1) / gridDim.x;
    const int grp = lane / G, gl = lane % G;

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
            acc_t acc[G];
#pragma unroll
            for (int t = 0; t < G; ++t) acc[t] = (acc_t)0;
#pragma unroll
            for (int t0 = 0; t0 < G; t0 += R) {
                const unsigned char *p[R];
                bool ok[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int in_batch = grp * G + t0 + r;
                    const long long rr = row0 + in_batch;
                    ok[r] = rr < a.n;
                    long long srow = rr;
                    if (a.slots != nullptr) srow = __shfl_sync(0xffffffffu, myslot, in_batch);
                    p[r] = a.rows + (ok[r] ? srow : 0) * a.ld;
                }
#pragma unroll 2
                for (int j = gl; j < a.chunks; j += G) {
                    const typename TR::QChunk qc = TR::load_q(qs, j, a.chunks);
                    int4 v[R];
#pragma unroll
                    for (int r = 0; r < R; ++r)
                        v[r] = ok[r] ? ld_stream16(p[r] + (size_t)j * 16) : make_int4(0, 0, 0, 0);
#pragma unroll
                    for (int r = 0; r < R; ++r) TR::dot(acc[t0 + r], v[r], qc);
                }
            }
            // transposed butterfly: lane i of the group ends with the total of row i
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
            const long long rr = row0 + lane;
            const bool valid = rr < a.n;
            const unsigned slot = (a.slots != nullptr) ? (unsigned)myslot : (unsigned)rr;
            unsigned long long key = 0ull;
            if (valid) key = make_key(TR::finish(acc[0], a, slot), slot);
            const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
            cand_offer_warp(buf, valid && key > thr && key < bound, key);
            b += kScanWarps;
            continue;
        }
        if (!work && !counted) {
            if (lane == 0) atomicAdd(&buf.ctrl->n_done, 1);
            counted = true;
        }
        __syncthreads();  // nobody appends past this point
        const int c = buf.ctrl->count, nd = buf.ctrl->n_done;
        __syncthreads();  // everybody has read the same state
        if (c > buf.limit || nd == kScanWarps) cand_prune(buf);
        if (nd == kScanWarps) break;
    }

    // ---- publish this CTA's list; the last CTA to arrive merges all lists ----
    unsigned long long *mine = a.part + (size_t)blockIdx.x * a.k;
    for (int i = tid; i < a.k; i += kScanThreads) mine[i] = buf.keys[i];
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    cand_select_from_global(buf, a.part, (long long)gridDim.x * a.k);
    const int cnt = buf.ctrl->count;
    for (int i = tid; i < a.k; i += kScanThreads) {
        const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
        a.out_keys[i] = key;
        float dq = 0.0f;
        if (TYPE == SCAN_I8 && key != 0ull) dq = a.qscale * a.scales[key_slot(key)];
        emit_hit(TYPE, key, i, a.shard_base, dq, a.out_ids, a.out_scores, a.out_iscores);
    }
    if (tid == 0) {
        *a.out_count = cnt;
        *a.ticket = 0u;
    }
}

// ---------------------------------------------------------------------------
// Merge of ranked lists (after the all-gather of per-shard candidates)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kScanThreads, 1) k_merge_lists(const MergeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
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
    cand_select_from_global(buf, scratch, total);
    const int cnt = buf.ctrl->count;
    for (int i = tid; i < a.k; i += kScanThreads) {
        const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
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

static size_t scan_smem_bytes(int type, int chunks, int k) {
    const int qb = (type == SCAN_I8) ? TraitsI8::kQBytes : (type == SCAN_F32 ? TraitsF32::kQBytes : TraitsF16::kQBytes);
    return (size_t)cand_capacity(k) * 8 + 16 + (size_t)chunks * qb;
}

typedef void (*scan_fn)(const ScanArgs);

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

int scan_resident_grid(int type, int chunks, int k, int device, int *err) {
    *err = 0;
    scan_fn fn = pick(type, scan_group_width(chunks));
    const size_t smem = scan_smem_bytes(type, chunks, k);
    cudaError_t e = cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { *err = (int)e; return 0; }
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void *)fn, kScanThreads, smem);
    if (e != cudaSuccess) { *err = (int)e; return 0; }
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) { *err = (int)e; return 0; }
    if (per_sm < 1) per_sm = 1;
    return per_sm * sms;
}

int scan_launch(int type, const ScanArgs &a, int grid, cudaStream_t stream) {
    scan_fn fn = pick(type, scan_group_width(a.chunks));
    const size_t smem = scan_smem_bytes(type, a.chunks, a.k);
    // never launch more CTAs than there are batches to hand out
    const long long batches = (a.n + 31) / 32;
    if (batches < grid) grid = (int)(batches > 0 ? batches : 1);
    fn<<<grid, kScanThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("scan launch: ") + cudaGetErrorString(e));
    return 0;
}

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
