// Device-side building blocks shared by every kernel of the KANLinear path:
// knot-span search, the k+1 non-zero B-spline values (and derivatives) of one
// input, SiLU and its derivative.
//
// Conventions (identical to the dense Cox-de Boor recurrence of the reference,
// spline_kan/reference_backend.py:69-94):
//   * spans are half-open [t_m, t_{m+1}); the last span is closed on the right;
//   * x outside [t_0, t_{T-1}] and NaN give an all-zero basis;
//   * a recurrence term whose knot difference is zero contributes zero, so
//     repeated knots are allowed.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace kanb200 {

constexpr int kMaxOrder = 3;
constexpr int kMaxKnots = 72;          // G + 2k + 1 <= 72  (G + 2k <= 71)

// Index m in [0, nk-2] of the knot span that holds x, or -1 when x lies
// outside the knot range (or is NaN).  x == t[nk-1] belongs to the last span.
template <typename T>
__device__ __forceinline__ int find_span(const T* __restrict__ t, int nk, T x) {
    if (!(x >= t[0]) || !(x <= t[nk - 1])) return -1;
    if (x == t[nk - 1]) return nk - 2;
    int lo = 0, hi = nk - 1;           // t[lo] <= x < t[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (t[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

// Quotient used inside the recurrence: IEEE division for double, the 2-ulp reciprocal-multiply
// for float (the float kernels are compared at 1e-5, the double ones at 1e-12).
template <typename T> __device__ __forceinline__ T ratio(T a, T b) { return a / b; }
template <> __device__ __forceinline__ float ratio<float>(float a, float b) { return __fdividef(a, b); }

// The K+1 basis functions that can be non-zero on span m are B_{m-K+j,K},
// j = 0..K.  val[j] receives their values at x; with DERIV, der[j] receives
// d/dx.  Built bottom-up over the degree (triangular de Boor table); knot
// reads beyond either end are clamped -- they only feed table entries that do
// not correspond to a real basis function and are dropped by the caller.
template <int K, typename T, bool DERIV>
__device__ __forceinline__ void local_basis(const T* __restrict__ t, int nk, int m, T x,
                                            T (&val)[K + 1], T (&der)[K + 1]) {
    auto knot = [&](int idx) -> T {
        idx = idx < 0 ? 0 : (idx > nk - 1 ? nk - 1 : idx);
        return t[idx];
    };
    T tk[2 * K];                        // t[m-K+1 .. m+K]
#pragma unroll
    for (int q = 0; q < 2 * K; ++q) tk[q] = knot(m - K + 1 + q);
    // tk index of knot t[m + d] is (K - 1 + d).
    T nd[K + 1];
    nd[0] = T(1);
#pragma unroll
    for (int j = 1; j <= K; ++j) nd[j] = T(0);
#pragma unroll
    for (int d = 1; d <= K; ++d) {
        if (DERIV && d == K) {
            // nd[0..K-1] hold the degree K-1 values B_{m-K+1+j, K-1}.
#pragma unroll
            for (int j = 0; j <= K; ++j) {
                T a = T(0), b = T(0);
                if (j >= 1) {           // B_{r,K-1}/(t_{r+K}-t_r), r = m-K+j
                    const T den = tk[K - 1 + j] - tk[j - 1];
                    if (den != T(0)) a = ratio<T>(nd[j - 1], den);
                }
                if (j <= K - 1) {       // B_{r+1,K-1}/(t_{r+K+1}-t_{r+1})
                    const T den = tk[K + j] - tk[j];
                    if (den != T(0)) b = ratio<T>(nd[j], den);
                }
                der[j] = T(K) * (a - b);
            }
        }
        T carry = T(0);
#pragma unroll
        for (int j = 0; j < d; ++j) {
            const T hi_k = tk[K + j];               // t[m + j + 1]
            const T lo_k = tk[K - d + j];           // t[m + 1 - d + j]
            const T den = hi_k - lo_k;
            const T w = (den != T(0)) ? ratio<T>(nd[j], den) : T(0);
            nd[j] = carry + (hi_k - x) * w;
            carry = (x - lo_k) * w;
        }
        nd[d] = carry;
    }
#pragma unroll
    for (int j = 0; j <= K; ++j) val[j] = nd[j];
}

// Places the K+1 local values of span m into a window of K+1 consecutive basis
// indices that lies inside [0, R-1].  Returns the window start; entries that do
// not correspond to a real basis function are zero.  m < 0 gives all zeros.
template <int K, typename T>
__device__ __forceinline__ int window_in_range(int m, int R, const T (&v)[K + 1], T (&w)[K + 1]) {
    if (m < 0) {
#pragma unroll
        for (int j = 0; j <= K; ++j) w[j] = T(0);
        return 0;
    }
    const int first = m - K;
    int s = first < 0 ? 0 : first;
    if (s > R - 1 - K) s = R - 1 - K;
    const int shift = s - first;        // in [-K, K]
#pragma unroll
    for (int j = 0; j <= K; ++j) {
        T pick = T(0);
#pragma unroll
        for (int q = 0; q <= K; ++q) pick = (q == j + shift) ? v[q] : pick;
        w[j] = pick;
    }
    return s;
}

template <typename T> __device__ __forceinline__ T sigmoid_t(T x);
template <> __device__ __forceinline__ float sigmoid_t<float>(float x) { return 1.0f / (1.0f + expf(-x)); }
template <> __device__ __forceinline__ double sigmoid_t<double>(double x) { return 1.0 / (1.0 + exp(-x)); }

template <typename T> __device__ __forceinline__ T silu_t(T x) { return x * sigmoid_t<T>(x); }
// sigma(x) (1 + x (1 - sigma(x)))
template <typename T> __device__ __forceinline__ T silu_grad_t(T x) {
    const T s = sigmoid_t<T>(x);
    return s * (T(1) + x * (T(1) - s));
}

}  // namespace kanb200
