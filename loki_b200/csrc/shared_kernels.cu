// Shared-concept ("must match all") scan: every stored row is scored against
// several query-side vectors at once, followed by a per-row scalar epilogue, fused
// with the same top-k selection as the single-query scan.
//
// Device replacement for
//   SharedQuery.Scorer       media-server/embedvec/shared.go:180-220
//   the centered wrapper     media-server/embedindex/embedindex.go:374-393
// The query-side preparation (normalise, centre, Gram-Schmidt basis, projected
// norms) is O(terms^2 * dim) and stays on the host (hostmath.hpp).
//
// Shape: a skinny matrix product  rows[N x dim] * terms[dim x T], T <= 32, with
// float64 accumulation like the reference.  This file holds the gathering kernel, used
// for allow-list scans (rows picked by slot) and for small indexes: a warp handles R
// rows at a time, lane l reads 16-byte chunks l, l+32, ... of each row straight from
// global memory and keeps R x T partial sums; the terms live in shared memory as float64.
// Scans over all rows of a larger index run on the float64 tensor-core kernel in
// shared_mma.cu, which this file's launcher tries first.
#include <algorithm>

#include "lk_common.cuh"
#include "shared.cuh"
#include "topk.cuh"

namespace lk {

template <int TP>  // TP = power of two >= number of terms
__global__ void __launch_bounds__(kScanThreads, 1) k_scan_shared(const SharedArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int R = (32 / TP) < 4 ? (32 / TP < 1 ? 1 : 32 / TP) : 4;
    constexpr int NV = R * TP;  // accumulators per lane
    CandBuf buf;
    buf.k = a.k;
    buf.cap = cand_capacity(a.k);
    buf.limit = buf.cap - kScanThreads;
    buf.keys = reinterpret_cast<unsigned long long *>(smem);
    buf.ctrl = reinterpret_cast<CandCtrl *>(smem + (size_t)buf.cap * 8);
    double2 *qs = reinterpret_cast<double2 *>(smem + (size_t)buf.cap * 8 + 16);
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const SharedParams &P = *a.params;
    const int T = P.m + P.rank + P.nneg;
    for (int i = tid; i < buf.cap; i += kScanThreads) buf.keys[i] = 0ull;
    if (tid == 0) {
        buf.ctrl->count = 0;
        buf.ctrl->n_done = 0;
        buf.ctrl->thr = a.floor ? __ldcg(a.floor) : 0ull;
    }
    // terms -> float64, two planes per term (elements 0,1 / 2,3 of each chunk)
    for (int i = tid; i < T * a.chunks; i += kScanThreads) {
        const int t = i / a.chunks, j = i % a.chunks;
        const float4 f = reinterpret_cast<const float4 *>(a.terms)[i];
        qs[(size_t)t * 2 * a.chunks + j] = make_double2((double)f.x, (double)f.y);
        qs[(size_t)t * 2 * a.chunks + a.chunks + j] = make_double2((double)f.z, (double)f.w);
    }
    const unsigned long long bound = a.bound ? __ldcg(a.bound) : ~0ull;
    __syncthreads();

    const long long n_batches = (a.n + R - 1) / R;
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
            const long long row0 = b * R;
            const unsigned char *p[R];
            bool ok[R];
            unsigned slot[R];
            float inv[R];
            bool dead[R];  // centered row sitting on the mean: scores 0
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const long long rr = row0 + r;
                ok[r] = rr < a.n;
                slot[r] = ok[r] ? (a.slots ? (unsigned)a.slots[rr] : (unsigned)rr) : 0u;
                p[r] = a.rows + (size_t)slot[r] * a.ld;
                inv[r] = 1.0f;
                dead[r] = false;
                if (a.cnorm != nullptr && ok[r]) {
                    const float cn = a.cnorm[slot[r]];
                    dead[r] = cn < 1e-6f;
                    inv[r] = dead[r] ? 0.0f : __fdiv_rn(1.0f, cn);
                }
            }
            double acc[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[i] = 0.0;
            for (int j = lane; j < a.chunks; j += 32) {
                double x[R][4];
                float4 m4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (a.cnorm != nullptr) m4 = reinterpret_cast<const float4 *>(a.mu)[j];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int4 v = ok[r] ? ld_stream16(p[r] + (size_t)j * 16) : make_int4(0, 0, 0, 0);
                    float f0 = __int_as_float(v.x), f1 = __int_as_float(v.y);
                    float f2 = __int_as_float(v.z), f3 = __int_as_float(v.w);
                    if (a.cnorm != nullptr) {  // (v - mu) * (1/cnorm), each step rounded to float32
                        f0 = __fmul_rn(__fsub_rn(f0, m4.x), inv[r]);
                        f1 = __fmul_rn(__fsub_rn(f1, m4.y), inv[r]);
                        f2 = __fmul_rn(__fsub_rn(f2, m4.z), inv[r]);
                        f3 = __fmul_rn(__fsub_rn(f3, m4.w), inv[r]);
                    }
                    x[r][0] = (double)f0;
                    x[r][1] = (double)f1;
                    x[r][2] = (double)f2;
                    x[r][3] = (double)f3;
                }
#pragma unroll
                for (int t = 0; t < TP; ++t) {
                    if (t < T) {
                        const double2 qa = qs[(size_t)t * 2 * a.chunks + j];
                        const double2 qb = qs[(size_t)t * 2 * a.chunks + a.chunks + j];
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            double s = acc[r * TP + t];
                            s = fma(x[r][0], qa.x, s);
                            s = fma(x[r][1], qa.y, s);
                            s = fma(x[r][2], qb.x, s);
                            s = fma(x[r][3], qb.y, s);
                            acc[r * TP + t] = s;
                        }
                    }
                }
            }
            // reduce across the warp; lane i (< NV) ends with the total of accumulator i
#pragma unroll
            for (int w = 16; w >= NV; w >>= 1) {
#pragma unroll
                for (int i = 0; i < NV; ++i)
                    acc[i] += __longlong_as_double((long long)shfl_xor_u64((uint64_t)__double_as_longlong(acc[i]), w));
            }
#pragma unroll
            for (int w = NV / 2; w >= 1; w >>= 1) {
                const bool upper = (lane & w) != 0;
#pragma unroll
                for (int i = 0; i < w; ++i) {
                    const double send = upper ? acc[i] : acc[i + w];
                    const double keep = upper ? acc[i + w] : acc[i];
                    acc[i] = keep + __longlong_as_double((long long)shfl_xor_u64((uint64_t)__double_as_longlong(send), w));
                }
            }
            // lane r*TP collects the T dots of row r (each rounded to float32 like embedvec.Cosine)
            const int my_r = (lane % NV) / TP;
            float dots[TP];
#pragma unroll
            for (int t = 0; t < TP; ++t) {
                const double v = __longlong_as_double((long long)__shfl_sync(
                    0xffffffffu, (unsigned long long)__double_as_longlong(acc[0]), my_r * TP + t));
                dots[t] = (float)v;
            }
            const bool head = lane < NV && (lane % TP) == 0;
            bool pass = false;
            unsigned long long key = 0ull;
            if (head) {
                bool okr = false, deadr = false;
                unsigned sl = 0;
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (r == my_r) { okr = ok[r]; deadr = dead[r]; sl = slot[r]; }
                if (okr) {
                    float out = 0.0f;
                    if (!deadr) {
                        // media-server/embedvec/shared.go:186-218
                        double b2 = 0.0;
#pragma unroll
                        for (int t = 0; t < TP; ++t)
                            if (t >= P.m && t < P.m + P.rank) b2 += (double)dots[t] * (double)dots[t];
                        double vn2 = __dsub_rn(1.0, __dmul_rn((double)P.gamma, b2));
                        if (vn2 < 1e-6) vn2 = 1e-6;
                        const double vn = sqrt(vn2);
                        double mean = 0.0, m2 = 0.0;
                        double sc[TP];
#pragma unroll
                        for (int i = 0; i < TP; ++i) {
                            sc[i] = 0.0;
                            if (i < P.m) {
                                double s = (double)dots[i];
#pragma unroll
                                for (int t = 0; t < TP; ++t)
                                    if (t >= P.m && t < P.m + P.rank)
                                        s = __dsub_rn(s, __dmul_rn(__dmul_rn((double)P.gamma, (double)P.qb[i * P.rank + (t - P.m)]),
                                                                   (double)dots[t]));
                                s = s / __dmul_rn((double)P.posnorm[i], vn);
                                sc[i] = s;
                                mean = __dadd_rn(mean, __dmul_rn((double)P.posw[i], s));
                            }
                        }
#pragma unroll
                        for (int i = 0; i < TP; ++i)
                            if (i < P.m) {
                                const double dd = sc[i] - mean;
                                m2 = __dadd_rn(m2, __dmul_rn(__dmul_rn((double)P.posw[i], dd), dd));
                            }
                        double o = __dsub_rn(mean, __dmul_rn((double)P.lambda, sqrt(m2)));
#pragma unroll
                        for (int t = 0; t < TP; ++t)
                            if (t >= P.m + P.rank && t < T)
                                o = __dsub_rn(o, __dmul_rn((double)P.negw[t - P.m - P.rank], (double)dots[t]));
                        out = (float)o;
                    }
                    key = make_key(ord_from_f32(out), sl);
                    const unsigned long long thr = *(volatile unsigned long long *)&buf.ctrl->thr;
                    pass = key > thr && key < bound;
                }
            }
            cand_offer_warp(buf, pass, key);
            b += kScanWarps;
            continue;
        }
        if (!work && !counted) {
            if (lane == 0) atomicAdd(&buf.ctrl->n_done, 1);
            counted = true;
        }
        __syncthreads();
        const int c = buf.ctrl->count, nd = buf.ctrl->n_done;
        __syncthreads();
        if (c > buf.limit || nd == kScanWarps) cand_prune(buf);
        if (nd == kScanWarps) break;
    }

    unsigned long long *mine = a.part + (size_t)blockIdx.x * a.k;
    for (int i = tid; i < a.k; i += kScanThreads) mine[i] = buf.keys[i];
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    cand_select_from_lists(buf, a.part, (int)gridDim.x);
    const int cnt = buf.ctrl->count;
    for (int i = tid; i < a.k; i += kScanThreads) {
        const unsigned long long key = (i < cnt) ? buf.keys[i] : 0ull;
        a.out_keys[i] = key;
        a.out_ids[i] = key ? a.shard_base + (long long)key_slot(key) : -1;
        a.out_scores[i] = key ? f32_from_ord(key_ord(key)) : 0.0f;
        if (a.out_iscores) a.out_iscores[i] = 0;
    }
    if (tid == 0) {
        *a.out_count = cnt;
        *a.ticket = 0u;
    }
}

typedef void (*shared_fn)(const SharedArgs);

static shared_fn pick_shared(int terms) {
    if (terms <= 1) return k_scan_shared<1>;
    if (terms <= 2) return k_scan_shared<2>;
    if (terms <= 4) return k_scan_shared<4>;
    if (terms <= 8) return k_scan_shared<8>;
    if (terms <= 16) return k_scan_shared<16>;
    return k_scan_shared<32>;
}

static size_t shared_smem(int terms, int chunks, int k) {
    return (size_t)cand_capacity(k) * 8 + 16 + (size_t)terms * chunks * 32;
}

constexpr size_t kShSmemLimit = 220 * 1024;

int shared_scan_grid(int terms, int chunks, int k, int device, int *err) {
    *err = 0;
    int sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) { *err = (int)e; return 0; }
    const size_t smem = shared_smem(terms, chunks, k);
    if (smem > kShSmemLimit) {
        // too many terms to keep widened beside the candidates: only the tensor-core kernel
        // (float32 terms, one CTA per SM) can take them
        if (!shared_mma_fits(terms, (long long)chunks * 16, k)) { *err = -1; return 0; }
        return sms;
    }
    shared_fn fn = pick_shared(terms);
    e = cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { *err = (int)e; return 0; }
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void *)fn, kScanThreads, smem);
    if (e != cudaSuccess) { *err = (int)e; return 0; }
    if (per_sm < 1) per_sm = 1;
    return per_sm * sms;
}

int shared_scan_launch(const SharedArgs &a, int terms, int grid, cudaStream_t stream) {
    const bool old_fits = shared_smem(terms, a.chunks, a.k) <= kShSmemLimit;
    // whole contiguous rows and enough of them: the float64 tensor-core kernel, one CTA per SM
    if (a.slots == nullptr && (a.n >= 8192 || !old_fits)) {
        const int st = shared_mma_launch(a, terms, grid, stream);
        if (st != 1) return st;
    }
    if (!old_fits) return fail(7, "shared scan: terms x dim too large for this scan");
    shared_fn fn = pick_shared(terms);
    const size_t smem = shared_smem(terms, a.chunks, a.k);
    if (a.n < grid) grid = (int)(a.n > 0 ? a.n : 1);
    fn<<<grid, kScanThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(4, std::string("shared scan launch: ") + cudaGetErrorString(e));
    return 0;
}

}  // namespace lk
