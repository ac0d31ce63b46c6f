// fp64 tensor-core multiply-accumulate (DMMA) for sm_100a.
//
// The 5th-generation tensor-core path (tcgen05) has no fp64 kind; fp64 matrix products go
// through warp-level mma.sync.  Measured on B200: 37.2 TFLOP/s with m8n8k4, against
// 34.1 TFLOP/s for a pure DFMA chain, the two sharing one pipe.
//
// m8n8k4 fragment layout (lane = 4*g + t, g = 0..7, t = 0..3):
//   A (8x4, row):  a    = A[g][t]
//   B (4x8, col):  b    = B[t][g]
//   C (8x8):       c[0] = C[g][2t], c[1] = C[g][2t+1]
#ifndef ACRO_B200_KERNELS_DMMA_CUH
#define ACRO_B200_KERNELS_DMMA_CUH

namespace acro_b200_detail
{

__device__ __forceinline__ void dmma_m8n8k4(double (&c)[2], double a, double b)
{
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c[0]), "+d"(c[1])
                 : "d"(a), "d"(b));
}

}

#endif
