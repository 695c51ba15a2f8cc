// Building blocks of the float64 tensor-core kernels (mma.sync m8n8k4 f64): operand loads
// from shared memory, the MMA itself, the group of MMAs that multiplies 16 floats of 8 rows
// with 8 NT right-hand vectors, and the mbarrier / bulk-copy forms that take 32-bit shared
// addresses.  Used by the shared-concept scan (shared_mma.cu) and the batched float32 scan
// (multi_mma.cu).
//
// Operand layout.  Lane (g = lane / 4, kq = lane % 4) reads 4 consecutive floats at element
// 16 c + 4 kq of left row g and feeds float i to MMA step i; the right-hand operand is read at
// the same positions of vector 8 nt + g, so each MMA step pairs matching elements.  With row
// pitches of 64 mod 128 bytes (float32) or 16 mod 128 bytes (float64 vectors) the 16-byte
// reads of a quarter warp fall in distinct banks.
#pragma once
#include <cuda_runtime.h>

namespace lk {

// Smallest pitch >= bytes (a multiple of 16) that is `mod` modulo 128.
__host__ __device__ inline long long mma_pitch(long long bytes, int mod) {
    long long p = bytes;
    while ((p & 127) != mod) p += 16;
    return p;
}
__device__ __forceinline__ void dmma_8x8x4(double &c0, double &c1, double a, double b) {
    asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}

// Shared-memory loads from a 32-bit address plus a compile-time offset (no address
// arithmetic in the unrolled multiply loop).  volatile: the buffers are rewritten by
// asynchronous copies, so a load must not be merged with one from an earlier slice.
template <int IMM>
__device__ __forceinline__ float4 lds_f4(unsigned addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr), "n"(IMM));
    return v;
}
template <int IMM>
__device__ __forceinline__ double2 lds_d2(unsigned addr) {
    double2 v;
    asm volatile("ld.shared.v2.f64 {%0,%1}, [%2+%3];" : "=d"(v.x), "=d"(v.y) : "r"(addr), "n"(IMM));
    return v;
}
__device__ __forceinline__ void mbar_expect_tx_u32(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_u32(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load_u32(unsigned dst, const void *src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// One group: 16 floats of each of the 8 rows against 8 NT terms = 4 NT MMAs.  Lane (g, kq)
// holds floats 4 kq .. 4 kq + 3 of row g and the same positions of its term row in each block.
template <int NT, bool F64T, bool CEN, int IMM>
__device__ __forceinline__ void mma_group(double (&acc)[NT][2][2], unsigned a_addr, unsigned m_addr, unsigned t_addr,
                                          const unsigned (&trow_off)[NT], float inv, bool in) {
    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
    if (in) {
        f = lds_f4<IMM>(a_addr);
        if (CEN) {  // (v - mu) * (1/cnorm), each step rounded to float32
            const float4 m4 = lds_f4<IMM>(m_addr);
            f.x = __fmul_rn(__fsub_rn(f.x, m4.x), inv);
            f.y = __fmul_rn(__fsub_rn(f.y, m4.y), inv);
            f.z = __fmul_rn(__fsub_rn(f.z, m4.z), inv);
            f.w = __fmul_rn(__fsub_rn(f.w, m4.w), inv);
        }
    }
    const double a0 = (double)f.x, a1 = (double)f.y, a2 = (double)f.z, a3 = (double)f.w;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        double b0 = 0.0, b1 = 0.0, b2 = 0.0, b3 = 0.0;
        if (in) {
            if (F64T) {
                const double2 x = lds_d2<2 * IMM>(t_addr + trow_off[nt]);
                const double2 y = lds_d2<2 * IMM + 16>(t_addr + trow_off[nt]);
                b0 = x.x; b1 = x.y; b2 = y.x; b3 = y.y;
            } else {
                const float4 q = lds_f4<IMM>(t_addr + trow_off[nt]);
                b0 = (double)q.x; b1 = (double)q.y; b2 = (double)q.z; b3 = (double)q.w;
            }
        }
        dmma_8x8x4(acc[nt][0][0], acc[nt][0][1], a0, b0);
        dmma_8x8x4(acc[nt][1][0], acc[nt][1][1], a1, b1);
        dmma_8x8x4(acc[nt][0][0], acc[nt][0][1], a2, b2);
        dmma_8x8x4(acc[nt][1][0], acc[nt][1][1], a3, b3);
    }
}

}  // namespace lk
