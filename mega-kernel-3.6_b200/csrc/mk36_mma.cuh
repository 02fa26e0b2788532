// Warp-level tensor-core helpers shared by the decode kernels: mma.sync.m16n8k16 with fp32
// accumulation and the fragment convention that lets every operand be fetched with one 128-bit load.
#pragma once

#include "mk36_common.cuh"

namespace mk36 {

#if defined(__CUDACC__)

// D += A(16x16, row) * B(16x8, col), fp32 accumulate
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                                  unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One 32-wide slice of the contraction for a 16 x 8 tile.  Lane (g = lane / 4, t = lane % 4) reads
// the 8 consecutive elements kb + 8t .. kb + 8t + 7 of its rows (A: rows g and g + 8; B: column g)
// with one 128-bit load each.  The contraction index is permuted the same way on both sides
// (elements 0,1 | 2,3 feed the first MMA's k slots 2t,2t+1 | 2t+8,2t+9; elements 4,5 | 6,7 the
// second MMA's), which leaves the sum unchanged and needs no shuffles or ldmatrix.
template <typename T>
__device__ __forceinline__ void mma_slice32(float (&d0)[4], float (&d1)[4], const uint4& a_lo, const uint4& a_hi, const uint4& b) {
    mma_16816<T>(d0, a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
    mma_16816<T>(d1, a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
}

#endif  // __CUDACC__

}  // namespace mk36
