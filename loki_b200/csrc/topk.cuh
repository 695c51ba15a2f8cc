// Exact top-k selection inside a CTA, fused into the kernels that produce scores.
//
// Every scoring kernel turns a score into a 64-bit ranking key (lk_common.cuh) and
// offers it to a per-CTA candidate buffer in shared memory.  A key is stored only
// if it beats the CTA's current threshold (the k-th best key seen so far), so after
// a short warm-up almost every row costs one compare.  When the buffer runs full
// the CTA sorts it (a bitonic network held in registers, see block_sort_desc), keeps the best k and raises the
// threshold.  Scores therefore never travel to HBM: a CTA writes k keys at the end,
// and the last CTA to finish merges all CTAs' lists with the same machinery.
//
// This replaces the reference's "materialise N float32 scores, then run a serial
// size-k min-heap over them" (media-server/embedindex/embedindex.go:432, :495-534)
// and its final sort (media-server/embedindex/embedindex.go:483-490).
#pragma once
#include "lk_common.cuh"

namespace lk {

constexpr int kScanThreads = 256;           // most threads any selecting CTA has (sizes the buffer slack)
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kMaxK = 2048;                 // largest k one pass selects; larger k runs more passes

// Buffer capacity for a given k: room for k survivors plus one full round of
// appends from every warp (32 keys each) after the "nearly full" mark is passed.
__host__ __device__ inline int cand_capacity(int k) {
    int need = k + kScanThreads;
    int cap = 512;
    while (cap < need) cap <<= 1;
    return cap;
}

struct CandCtrl {
    int count;               // keys currently in the buffer
    int n_done;              // warps that have no rows left
    unsigned long long thr;  // keys must be strictly greater than this to enter
};

struct CandBuf {
    unsigned long long *keys;  // [cap] shared memory
    CandCtrl *ctrl;            // shared memory
    int cap;
    int limit;                 // prune once count exceeds this (= cap - kScanThreads)
    int k;
};

// ---------------------------------------------------------------------------
// Bitonic sort (descending) of sz keys in shared memory by the whole CTA; sz is a power of two,
// at least kSortSegment.  The network's compare-exchanges between keys fewer than kSortSegment
// apart stay inside an aligned segment of 256 keys, and a warp does them with the segment in
// registers: lane l holds keys 8l..8l+7, partners 1, 2 or 4 apart meet in the lane's own registers
// and partners 8..128 apart through warp shuffles.  All phases up to 256 keys therefore need no
// barrier at all, and each later phase needs one barrier per stride of 256 and up plus one for
// its register part: 14 barriers for 2,048 keys, where a sort through shared memory takes 66.
// Not inlined: the network is a few thousand instructions, and the scan kernels exist in dozens of
// instantiations.  Every thread of the CTA calls it; the keys are visible to all threads on return.
// ---------------------------------------------------------------------------
constexpr int kSortSegment = 256;

__device__ __forceinline__ void sort_cx(unsigned long long &lo, unsigned long long &hi, bool desc) {
    const bool sw = (lo < hi) == desc;  // descending: the larger key belongs at the lower index
    const unsigned long long t = lo;
    lo = sw ? hi : lo;
    hi = sw ? t : hi;
}

// strides 4, 2, 1 (those not above FIRST) of phase `size` on a lane's eight keys; i0 = index of v[0]
template <int FIRST>
__device__ __forceinline__ void sort_reg_steps(unsigned long long (&v)[8], int i0, int size) {
#pragma unroll
    for (int stride = 4; stride > 0; stride >>= 1) {
        if (stride > FIRST) continue;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if ((e & stride) == 0) sort_cx(v[e], v[e + stride], ((i0 + e) & size) == 0);
    }
}

// strides 8*first, ..., 16, 8 of phase `size` (at least 16): partners sit in lanes first, ..., 2, 1 apart
__device__ __forceinline__ void sort_lane_steps(unsigned long long (&v)[8], int i0, int size, int first, int lane) {
    const bool desc = (i0 & size) == 0;  // the same for a lane's eight keys and for its partner's
    for (int ls = first; ls > 0; ls >>= 1) {
        const bool keep_larger = ((lane & ls) == 0) == desc;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const unsigned long long o = shfl_xor_u64(v[e], ls);
            v[e] = ((v[e] > o) == keep_larger) ? v[e] : o;
        }
    }
}

__device__ __noinline__ inline void block_sort_desc(unsigned long long *keys, int sz) {
    const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, warps = T >> 5;
    const unsigned base = (unsigned)__cvta_generic_to_shared(keys);
    auto load8 = [&](int i0, unsigned long long (&v)[8]) {
#pragma unroll
        for (int e = 0; e < 8; e += 2)
            asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v[e]), "=l"(v[e + 1]) : "r"(base + (unsigned)(i0 + e) * 8u));
    };
    auto store8 = [&](int i0, const unsigned long long (&v)[8]) {
#pragma unroll
        for (int e = 0; e < 8; e += 2)
            asm volatile("st.shared.v2.u64 [%2], {%0, %1};" ::"l"(v[e]), "l"(v[e + 1]), "r"(base + (unsigned)(i0 + e) * 8u) : "memory");
    };
    // phases 2 .. 256: whole segments, no barrier
    for (int seg = warp * kSortSegment; seg < sz; seg += warps * kSortSegment) {
        const int i0 = seg + lane * 8;
        unsigned long long v[8];
        load8(i0, v);
        sort_reg_steps<1>(v, i0, 2);
        sort_reg_steps<2>(v, i0, 4);
        sort_reg_steps<4>(v, i0, 8);
#pragma unroll 1
        for (int size = 16; size <= kSortSegment; size <<= 1) {
            sort_lane_steps(v, i0, size, size >> 4, lane);
            sort_reg_steps<4>(v, i0, size);
        }
        store8(i0, v);
    }
    __syncthreads();
    for (int size = 2 * kSortSegment; size <= sz; size <<= 1) {
        for (int stride = size >> 1; stride >= kSortSegment; stride >>= 1) {
            for (int i = tid; i < (sz >> 1); i += T) {
                const int pos = 2 * i - (i & (stride - 1));
                const unsigned pa = base + (unsigned)pos * 8u, pb = pa + (unsigned)stride * 8u;
                unsigned long long x, y;
                asm volatile("ld.shared.u64 %0, [%1];" : "=l"(x) : "r"(pa));
                asm volatile("ld.shared.u64 %0, [%1];" : "=l"(y) : "r"(pb));
                if ((x < y) == ((pos & size) == 0)) {
                    asm volatile("st.shared.u64 [%0], %1;" ::"r"(pa), "l"(y) : "memory");
                    asm volatile("st.shared.u64 [%0], %1;" ::"r"(pb), "l"(x) : "memory");
                }
            }
            __syncthreads();
        }
        for (int seg = warp * kSortSegment; seg < sz; seg += warps * kSortSegment) {
            const int i0 = seg + lane * 8;
            unsigned long long v[8];
            load8(i0, v);
            sort_lane_steps(v, i0, size, 16, lane);
            sort_reg_steps<4>(v, i0, size);
            store8(i0, v);
        }
        __syncthreads();
    }
}

// cand_prune for up to 32 R keys, by one warp: key i sits in register i / 32 of lane i % 32.  A bitonic
// network: partners up to 16 apart meet through shuffles, partners 32 and 64 apart in the lane's own
// registers.  Keeps the best k, zeroes the rest, raises the threshold.
// Not inlined (like block_sort_desc): cand_prune sits in dozens of kernel instantiations.
template <int R>
__device__ __noinline__ void warp_sort_prune(unsigned long long *keys, CandCtrl *ctrl, int k, int c, int lane) {
    unsigned long long v[R];
#pragma unroll
    for (int e = 0; e < R; ++e) v[e] = (e * 32 + lane < c) ? keys[e * 32 + lane] : 0ull;
#pragma unroll
    for (int size = 2; size <= 32 * R; size <<= 1) {
#pragma unroll
        for (int rs = R / 2; rs > 0; rs >>= 1) {  // strides of 32 rs keys: inside the lane
            if (32 * rs >= size) continue;
#pragma unroll
            for (int e = 0; e < R; ++e) {
                if ((e & rs) != 0) continue;
                const bool desc = ((e * 32) & size) == 0;
                const unsigned long long x = v[e], y = v[e + rs];
                const bool sw = (x < y) == desc;
                v[e] = sw ? y : x;
                v[e + rs] = sw ? x : y;
            }
        }
#pragma unroll
        for (int stride = 16; stride > 0; stride >>= 1) {
            if (stride >= size) continue;
            const bool lower = (lane & stride) == 0;
#pragma unroll
            for (int e = 0; e < R; ++e) {
                const bool desc = ((e * 32 + lane) & size) == 0;
                const unsigned long long o = shfl_xor_u64(v[e], stride);
                v[e] = ((v[e] > o) == (lower == desc)) ? v[e] : o;  // the lower lane of a descending pair keeps the larger key
            }
        }
    }
    const int keep = c < k ? c : k;
    unsigned long long kth = 0ull;
#pragma unroll
    for (int e = 0; e < R; ++e) {
        keys[e * 32 + lane] = (e * 32 + lane < keep) ? v[e] : 0ull;
        const unsigned long long at = shfl_u64(v[e], (k - 1) & 31);  // the k-th key, when there are k
        if (((k - 1) >> 5) == e) kth = at;
    }
    if (lane == 0) {
        ctrl->count = keep;
        if (keep == k && kth > ctrl->thr) ctrl->thr = kth;  // only ever rises
    }
}

// Sort keys[0..count) descending, keep the best k, zero the rest, raise thr.
// Must be called by all threads of the CTA with `count` stable.
__device__ inline void cand_prune(const CandBuf &b) {
    const int tid = threadIdx.x, T = blockDim.x;
    const int c = b.ctrl->count;
    if (c <= 128) {
        // few keys (a CTA's warps handing over their registers' best 10 at the end of a scan, a handful of
        // survivors of a bounded scan): one warp sorts them in registers, no barrier, little code
        if (tid < 32) {
            if (c <= 32) warp_sort_prune<1>(b.keys, b.ctrl, b.k, c, tid);
            else if (c <= 64) warp_sort_prune<2>(b.keys, b.ctrl, b.k, c, tid);
            else warp_sort_prune<4>(b.keys, b.ctrl, b.k, c, tid);
        }
        __syncthreads();
        return;
    }
    int sz = kSortSegment;  // (every buffer holds at least 512 keys)
    while (sz < c) sz <<= 1;
    for (int i = c + tid; i < sz; i += T) b.keys[i] = 0ull;
    __syncthreads();
    block_sort_desc(b.keys, sz);
    const int keep = c < b.k ? c : b.k;
    for (int i = keep + tid; i < sz; i += T) b.keys[i] = 0ull;
    if (tid == 0) {
        b.ctrl->count = keep;
        if (keep == b.k && b.keys[b.k - 1] > b.ctrl->thr) b.ctrl->thr = b.keys[b.k - 1];  // only ever rises
    }
    __syncthreads();
}

// Warp-aggregated append: lanes with pass==true store their key.  The caller has
// checked count <= limit before producing this batch, which leaves room for one
// batch from every warp.
__device__ __forceinline__ void cand_offer_warp(const CandBuf &b, bool pass, unsigned long long key) {
    const unsigned m = __ballot_sync(0xffffffffu, pass);
    if (m == 0) return;
    const int lane = threadIdx.x & 31;
    const int leader = __ffs(m) - 1;
    int base = 0;
    if (lane == leader) base = atomicAdd(&b.ctrl->count, __popc(m));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (pass) b.keys[base + __popc(m & lanemask_lt())] = key;
}

// ---------------------------------------------------------------------------
// Small k (<= 32): a warp keeps its own best keys in registers, lane i holding the i-th best
// (descending, 0 = none yet), and never touches the CTA's buffer or a barrier while it streams:
// the buffer's prune is a meeting of all warps, during which none of them has copies in flight.
// A batch's candidates are inserted one by one (a ballot gives the place, a shuffle makes room)
// when they are few, or sorted and merged as a whole (bitonic networks over the lanes) when many
// pass, as in the first batches.  `wthr` is the key at lane k-1, the warp's own threshold.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void warp_top_offer(unsigned long long &wk, unsigned long long &wthr, int k, bool pass,
                                               unsigned long long key, int lane) {
    unsigned m = __ballot_sync(0xffffffffu, pass);
    if (m == 0u) return;
    if (__popc(m) <= 4) {
        while (m != 0u) {  // warp-uniform
            const int src = __ffs(m) - 1;
            m &= m - 1u;
            const unsigned long long c = shfl_u64(key, src);
            if (c <= wthr) continue;  // an earlier insertion of this batch may have raised the threshold
            const int pos = __popc(__ballot_sync(0xffffffffu, wk > c));  // wk is descending: the lanes above c are a prefix
            const unsigned long long up = shfl_up_u64(wk, 1);
            wk = lane < pos ? wk : (lane == pos ? c : up);
            wthr = shfl_u64(wk, k - 1);
        }
        return;
    }
    unsigned long long c = pass ? key : 0ull;
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {  // sort the candidates, descending over the lanes
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const unsigned long long o = shfl_xor_u64(c, stride);
            const bool lower = (lane & stride) == 0, desc = (lane & size) == 0;
            c = ((c > o) == (lower == desc)) ? c : o;
        }
    }
    // best 32 of two descending runs: pair the i-th of one with the (31-i)-th of the other, keep the
    // larger (a bitonic sequence), then five merge steps
    const unsigned long long r = shfl_u64(c, 31 - lane);
    unsigned long long v = wk > r ? wk : r;
#pragma unroll
    for (int stride = 16; stride > 0; stride >>= 1) {
        const unsigned long long o = shfl_xor_u64(v, stride);
        const bool lower = (lane & stride) == 0;
        v = ((v > o) == lower) ? v : o;
    }
    wk = v;
    wthr = shfl_u64(wk, k - 1);
}

// Select the best k out of `lists` ranked lists of k keys each (global memory, zero
// padded, list l at src[l*k]) into the buffer, sorted descending.  All threads of
// the CTA call this in lockstep.
//
// Starting threshold.  Let p = ceil(k / lists) - 1 and j = ceil(k / (p+1)): the j-th
// largest of the lists' entries at position p has at least j*(p+1) >= k keys at or
// above it (p+1 from each of j lists), so it is a lower bound on the k-th best key
// overall and nearly every key fails its first compare against it.
//
// Keys are fetched kSelectUnroll per thread at a time with independent loads (one
// memory latency per round instead of one per key).  Should a round offer more keys
// than the buffer has room for, the buffer is pruned and the same registers are
// offered again, so nothing is ever dropped.
constexpr int kSelectUnroll = 16;

__device__ inline void cand_select_from_lists(const CandBuf &b, const unsigned long long *src, int lists,
                                              int stride = 0) {
    const int tid = threadIdx.x, T = blockDim.x;
    if (stride == 0) stride = b.k;  // list l starts at src[l * stride]; entries past k are ignored
    const long long total = (long long)lists * b.k;
    __shared__ int s_overflow;
    for (int i = tid; i < b.cap; i += T) b.keys[i] = 0ull;
    if (tid == 0) {
        b.ctrl->count = 0;
        b.ctrl->thr = 0ull;
        s_overflow = 0;
    }
    __syncthreads();
    if (lists <= b.cap) {
        const int p = (b.k + lists - 1) / lists - 1;
        const int j = (b.k + p) / (p + 1);
        for (int l = tid; l < lists; l += T) b.keys[l] = __ldcg(src + (size_t)l * stride + p);
        __syncthreads();
        for (int l = tid; l < lists; l += T) {
            const unsigned long long h = b.keys[l];
            int rank = 0;
            for (int m = 0; m < lists; ++m) rank += (b.keys[m] > h) ? 1 : 0;
            if (rank == j - 1 && h > 0ull) b.ctrl->thr = h - 1ull;  // keys are unique: one writer
        }
        __syncthreads();
        for (int l = tid; l < lists; l += T) b.keys[l] = 0ull;
        __syncthreads();
    }
    // Fast path: the lists are ranked, so the keys above the starting threshold are a
    // prefix of each list.  One thread per list finds its prefix length by bisection
    // (log2 k dependent loads instead of k); if all prefixes fit in the buffer together
    // they are copied in and one sort finishes the job.
    __shared__ int s_total;
    const unsigned long long thr0 = b.ctrl->thr;
    if (thr0 != 0ull) {
        if (tid == 0) s_total = 0;
        __syncthreads();
        for (int l0 = 0; l0 < lists; l0 += T) {
            const int l = l0 + tid;
            int cut = 0;
            if (l < lists) {
                const unsigned long long *lst = src + (size_t)l * stride;
                int lo = 0, hi = b.k;  // first index whose key is <= thr0 lies in [lo, hi]
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (__ldcg(lst + mid) > thr0) lo = mid + 1; else hi = mid;
                }
                cut = lo;
            }
            const int at = (cut > 0) ? atomicAdd(&s_total, cut) : 0;
            if (cut > 0 && at + cut <= b.cap) {
                const unsigned long long *lst = src + (size_t)l * stride;
                for (int i = 0; i < cut; ++i) b.keys[at + i] = __ldcg(lst + i);
            }
        }
        __syncthreads();
        const int tot = s_total;
        __syncthreads();
        if (tot <= b.cap) {
            if (tid == 0) b.ctrl->count = tot;
            __syncthreads();
            cand_prune(b);
            return;
        }
        // too many survivors for one buffer: start over with the streaming pass below
        for (int i = tid; i < b.cap; i += T) b.keys[i] = 0ull;
        __syncthreads();
    }
    for (long long base = 0; base < total; base += (long long)T * kSelectUnroll) {
        unsigned long long key[kSelectUnroll];
#pragma unroll
        for (int u = 0; u < kSelectUnroll; ++u) {
            const long long i = base + (long long)u * T + tid;
            key[u] = (i < total) ? __ldcg(src + (i / b.k) * stride + (i % b.k)) : 0ull;
        }
        for (;;) {
            const unsigned long long thr = *(volatile unsigned long long *)&b.ctrl->thr;
#pragma unroll
            for (int u = 0; u < kSelectUnroll; ++u) {
                if (key[u] > thr) {
                    const int pos = atomicAdd(&b.ctrl->count, 1);
                    if (pos < b.cap) {
                        b.keys[pos] = key[u];
                        key[u] = 0ull;
                    } else {
                        s_overflow = 1;  // keep the key in its register for the next attempt
                    }
                } else {
                    key[u] = 0ull;
                }
            }
            __syncthreads();
            const int c = b.ctrl->count;
            const int ov = s_overflow;
            __syncthreads();
            if (ov == 0) {
                if (c > b.limit) cand_prune(b);
                break;
            }
            if (tid == 0) {
                b.ctrl->count = b.cap;  // every slot below cap was written
                s_overflow = 0;
            }
            __syncthreads();
            cand_prune(b);
        }
    }
    cand_prune(b);
}

// The selection for small k (<= 32): no starting threshold to work out and no list lengths needed.
// One thread per list fetches the list's head chunk (one round trip for all lists); every warp then
// folds its 32 lists into a register-held best-k with warp_top_offer, position by position, and stops
// as soon as no lane's next key beats the warp's threshold (the lists are ranked, so nothing further
// down can); the warps' lists meet in the buffer for one small sort.  All threads of the CTA call this
// in lockstep.
__device__ inline void cand_select_small(const CandBuf &b, const unsigned long long *src, int lists, int stride = 0) {
    const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31;
    if (stride == 0) stride = b.k;
    for (int i = tid; i < b.cap; i += T) b.keys[i] = 0ull;
    if (tid == 0) {
        b.ctrl->count = 0;
        b.ctrl->thr = 0ull;
    }
    __syncthreads();
    unsigned long long wk = 0ull, wthr = 0ull;
    for (int l0 = 0; l0 < lists; l0 += T) {  // the same trip count for every thread
        const int l = l0 + tid;
        const unsigned long long *lst = src + (size_t)min(l, lists - 1) * stride;
        for (int base = 0; base < b.k; base += 8) {
            unsigned long long key[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) key[u] = (l < lists && base + u < b.k) ? __ldcg(lst + base + u) : 0ull;
            bool more = false;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                warp_top_offer(wk, wthr, b.k, key[u] > wthr, key[u], lane);
                more = key[u] > wthr;  // after the offer: does this list still reach into the warp's best k?
            }
            if (!__any_sync(0xffffffffu, more)) break;
        }
    }
    // the warps' lists meet in the buffer (warp w at [32w, 32w+32)); warp 0 folds them into its own
    const int warp = tid >> 5, nwarps = T >> 5;
    b.keys[warp * 32 + lane] = wk;
    __syncthreads();
    if (warp == 0) {
        for (int w = 1; w < nwarps; ++w) {
            const unsigned long long c = b.keys[w * 32 + lane];
            warp_top_offer(wk, wthr, b.k, c > wthr, c, lane);
        }
        const bool keep = lane < b.k && wk != 0ull;
        b.keys[lane] = keep ? wk : 0ull;
        const int cnt = __popc(__ballot_sync(0xffffffffu, keep));
        if (lane == 0) {
            b.ctrl->count = cnt;
            if (cnt == b.k) b.ctrl->thr = wthr;
        }
    }
    __syncthreads();
    for (int i = 32 + tid; i < nwarps * 32; i += T) b.keys[i] = 0ull;
    __syncthreads();
}

// The same selection without bisection, for when every list's length is known (cnts[l] keys, then
// zeros).  One round trip fetches every list's entry at position p (for the starting threshold, as
// above) together with the lengths; then one thread per list walks its list from the top in chunks
// of eight independent loads and keeps what beats the threshold, stopping at the first key that
// does not: the lists are ranked, so that is a prefix, usually inside the first chunk.  Returns
// false when more keys survive than the buffer holds (the caller then runs
// cand_select_from_lists, which starts over).  All threads of the CTA call this in lockstep.
__device__ inline bool cand_select_flat(const CandBuf &b, const unsigned long long *src, const int *cnts, int lists,
                                        int stride = 0) {
    const int tid = threadIdx.x, T = blockDim.x;
    if (stride == 0) stride = b.k;
    if (cnts == nullptr || lists > b.cap) return false;
    __shared__ int s_over;
    for (int i = tid; i < b.cap; i += T) b.keys[i] = 0ull;
    if (tid == 0) {
        b.ctrl->count = 0;
        b.ctrl->thr = 0ull;
        s_over = 0;
    }
    __syncthreads();
    const int p = (b.k + lists - 1) / lists - 1;
    const int j = (b.k + p) / (p + 1);
    for (int l = tid; l < lists; l += T) b.keys[l] = __ldcg(src + (size_t)l * stride + p);
    __syncthreads();
    for (int l = tid; l < lists; l += T) {
        const unsigned long long h = b.keys[l];
        int r0 = 0, r1 = 0, r2 = 0, r3 = 0;  // independent counts: the shared-memory reads overlap
        int m = 0;
        for (; m + 4 <= lists; m += 4) {
            r0 += (b.keys[m] > h) ? 1 : 0;
            r1 += (b.keys[m + 1] > h) ? 1 : 0;
            r2 += (b.keys[m + 2] > h) ? 1 : 0;
            r3 += (b.keys[m + 3] > h) ? 1 : 0;
        }
        for (; m < lists; ++m) r0 += (b.keys[m] > h) ? 1 : 0;
        const int rank = r0 + r1 + r2 + r3;
        if (rank == j - 1 && h > 0ull) b.ctrl->thr = h - 1ull;  // keys are unique: one writer
    }
    __syncthreads();
    for (int l = tid; l < lists; l += T) b.keys[l] = 0ull;
    __syncthreads();
    const unsigned long long thr0 = b.ctrl->thr;
    for (int l = tid; l < lists; l += T) {
        const unsigned long long *lst = src + (size_t)l * stride;
        const int c = min(__ldcg(cnts + l), b.k);  // (entries past the length are zero: the bound below is b.k,
        for (int base = 0; base < c; base += 8) {  //  so that the loads need not wait for the length)
            unsigned long long key[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) key[u] = (base + u < b.k) ? __ldcg(lst + base + u) : 0ull;
            int take = 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) take += (key[u] > thr0) ? 1 : 0;  // ranked: the takers come first
            if (take > 0) {
                const int at = atomicAdd(&b.ctrl->count, take);
                if (at + take <= b.cap) {
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (u < take) b.keys[at + u] = key[u];
                } else {
                    s_over = 1;
                }
            }
            if (take < 8) break;
        }
    }
    __syncthreads();
    if (s_over != 0) return false;
    cand_prune(b);
    return true;
}

}  // namespace lk
