// Shared device helpers: sortable 64-bit ranking keys, cache-hinted loads, error plumbing.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <string>

namespace lk {

// ---------------------------------------------------------------------------
// Ranking key.  One 64-bit word orders candidates exactly as the index promises:
// score descending, slot ascending on equal scores.
//   bits 63..32  order-preserving image of the score (int32 or float32)
//   bits 31..0   ~slot, so that among equal scores the lower slot has the larger key
// 0 is reserved for "no candidate"; every real key is > 0.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t ord_from_i32(int32_t s) {
    return (uint32_t)s ^ 0x80000000u;
}
__host__ __device__ __forceinline__ int32_t i32_from_ord(uint32_t o) {
    return (int32_t)(o ^ 0x80000000u);
}
// -0 is folded into +0 (the reference compares floats, so they tie); NaN ranks last.
__host__ __device__ __forceinline__ uint32_t ord_from_f32(float f) {
    if (f != f) return 0u;
    f = f + 0.0f;
#ifdef __CUDA_ARCH__
    uint32_t b = __float_as_uint(f);
#else
    uint32_t b;
    memcpy(&b, &f, 4);
#endif
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ __forceinline__ float f32_from_ord(uint32_t o) {
    uint32_t b = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    float f;
    memcpy(&f, &b, 4);
    return f;
#endif
}
__host__ __device__ __forceinline__ uint64_t make_key(uint32_t ord, uint32_t slot) {
    return ((uint64_t)ord << 32) | (uint64_t)(~slot);
}
__host__ __device__ __forceinline__ uint32_t key_slot(uint64_t k) { return ~(uint32_t)k; }
__host__ __device__ __forceinline__ uint32_t key_ord(uint64_t k) { return (uint32_t)(k >> 32); }

#ifdef __CUDACC__
// 16-byte streaming load of corpus data: read-only path, do not keep in L1.
__device__ __forceinline__ int4 ld_stream16(const void *p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t lanemask_lt() {
    uint32_t m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}
__device__ __forceinline__ uint64_t shfl_u64(uint64_t v, int src_lane) {
    uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
    lo = __shfl_sync(0xffffffffu, lo, src_lane);
    hi = __shfl_sync(0xffffffffu, hi, src_lane);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ uint64_t shfl_up_u64(uint64_t v, int delta) {
    uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
    lo = __shfl_up_sync(0xffffffffu, lo, delta);
    hi = __shfl_up_sync(0xffffffffu, hi, delta);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t v, int m) {
    uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
    lo = __shfl_xor_sync(0xffffffffu, lo, m);
    hi = __shfl_xor_sync(0xffffffffu, hi, m);
    return ((uint64_t)hi << 32) | lo;
}
#endif

// ---------------------------------------------------------------------------
// Host-side error plumbing.
// ---------------------------------------------------------------------------
void set_error(const std::string &msg);
int fail(int status, const std::string &msg);

#define LK_CUDA(expr)                                                                   \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess)                                                          \
            return lk::fail(4 /*LK_ECUDA*/, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

#define LK_TRY(expr)              \
    do {                          \
        int _s = (expr);          \
        if (_s != 0) return _s;   \
    } while (0)

__host__ __device__ static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

}  // namespace lk
