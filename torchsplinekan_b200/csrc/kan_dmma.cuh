// FP64 matrix instructions (mma.sync ... f64): the only FP64 matrix path of the part; tcgen05 has
// no FP64 kind.  Fragment layouts (lane = 4 * g + t, g = 0..7, t = 0..3):
//   m8n8k4   A[8x4]  a     = A[g][t]          B[4x8]  b     = B[t][g]
//            C[8x8]  c0,c1 = C[g][2t], C[g][2t+1]
//   m16n8k8  A[16x8] a0..3 = A[g][t], A[g+8][t], A[g][t+4], A[g+8][t+4]
//            B[8x8]  b0,b1 = B[t][g], B[t+4][g]
//            C[16x8] c0..3 = C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1]
#pragma once

namespace kanb200 {
namespace dmma {

__device__ __forceinline__ void m8n8k4(double& c0, double& c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}

__device__ __forceinline__ void m16n8k8(double (&c)[4], const double (&a)[4], const double (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
        : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

}  // namespace dmma
}  // namespace kanb200
