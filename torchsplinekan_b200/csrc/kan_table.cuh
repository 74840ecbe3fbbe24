// Per-span polynomial form of the B-spline basis, shared by the tensor-core operand producers
// (kan_tc.cu) and the table-driven basis kernels (kan_simt.cu).
//
// On a knot span [t_m, t_{m+1}) each of the k+1 non-zero basis functions is a polynomial of
// degree k in u = x - t_m.  poly_table_entry expands the de Boor recurrence symbolically (in
// double) and writes one 20-float entry: 16 coefficients c[j][p] (function j of the window,
// power p of u), t_m, the window start s = m - k (as int bits), 2 unused.  Coefficients of
// window slots outside [0, R) are zero; m == nk - 1 gives the all-zero entry that inputs outside
// the knot range select.  Conventions (half-open spans, last span closed, zero-length spans
// contribute zero) are those of the dense recurrence.
#pragma once
#include <cuda_runtime.h>

namespace kanb200 {

constexpr int TAB_ENTRY_FLOATS = 20;

__device__ inline void poly_table_entry(const float* __restrict__ t, int nk, int K, int R, int m,
                                        float* __restrict__ ent) {
    double c[4][4];
    for (int j = 0; j < 4; ++j)
        for (int p = 0; p < 4; ++p) c[j][p] = 0.0;
    float tm = 0.0f;
    int s = 0;
    if (m <= nk - 2) {
        auto knot = [&](int i) -> double { return (double)t[i < 0 ? 0 : (i > nk - 1 ? nk - 1 : i)]; };
        tm = t[m];
        s = m - K;
        c[0][0] = 1.0;
        for (int d = 1; d <= K; ++d) {
            double carry[4] = {0.0, 0.0, 0.0, 0.0};
            for (int j = 0; j < d; ++j) {
                const double hi_k = knot(m + j + 1), lo_k = knot(m + 1 - d + j);
                const double den = hi_k - lo_k;
                double w[4];
                for (int p = 0; p < 4; ++p) w[p] = (den != 0.0) ? c[j][p] / den : 0.0;
                // (hi_k - x) w = ((hi_k - t_m) - u) w ;  (x - lo_k) w = (u + (t_m - lo_k)) w
                const double a = hi_k - (double)tm, b = (double)tm - lo_k;
                double left[4], right[4];
                for (int p = 0; p < 4; ++p) {
                    const double wm1 = (p > 0) ? w[p - 1] : 0.0;
                    left[p] = a * w[p] - wm1;
                    right[p] = b * w[p] + wm1;
                }
                for (int p = 0; p < 4; ++p) {
                    c[j][p] = carry[p] + left[p];
                    carry[p] = right[p];
                }
            }
            for (int p = 0; p < 4; ++p) c[d][p] = carry[p];
        }
        for (int j = 0; j < 4; ++j) {
            const int r = s + j;
            if (j > K || r < 0 || r >= R)
                for (int p = 0; p < 4; ++p) c[j][p] = 0.0;
        }
    }
    for (int j = 0; j < 4; ++j)
        for (int p = 0; p < 4; ++p) ent[j * 4 + p] = (float)c[j][p];
    ent[16] = tm;
    ent[17] = __int_as_float(s);
    ent[18] = 0.0f;
    ent[19] = 0.0f;
}

// Knot block of a feature with at most 12 knots, for the compare-and-count span search:
// out[0..10] = t_0 .. t_{nk-2} padded with +inf, out[11] = t_{nk-1}.
__device__ inline void poly_table_knots12(const float* __restrict__ t, int nk, float* __restrict__ out) {
    for (int q = 0; q < 11; ++q) out[q] = (q <= nk - 2) ? t[q] : __int_as_float(0x7f800000);
    out[11] = t[nk - 1];
}

// Entry index for x from a 12-slot knot block (three 16-byte pieces): the knot span (last knot
// <= x; the last span is closed on the right) or nk - 1 (the all-zero entry) outside / NaN.
__device__ __forceinline__ int entry_index12(const float4& k0, const float4& k1, const float4& k2, int nk, float xv) {
    const bool inside = (xv >= k0.x) && (xv <= k2.w);
    const int m = (xv >= k0.y) + (xv >= k0.z) + (xv >= k0.w) + (xv >= k1.x) + (xv >= k1.y) + (xv >= k1.z) +
                  (xv >= k1.w) + (xv >= k2.x) + (xv >= k2.y) + (xv >= k2.z);
    return inside ? m : nk - 1;
}

}  // namespace kanb200
