// Device-side building blocks of the gather (FMA-pipe) kernels: knot-span search, the k+1 non-zero
// B-spline values (and derivatives) of one input evaluated in registers, SiLU and its derivative.
// (The tensor-core kernels and the table-driven basis kernels evaluate the same functions from the
// per-span polynomial table of kan_table.cuh instead.)
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

// Knot span of x: the largest m <= nk - 2 with t[m] <= x (so repeated knots select the span that
// follows them, and x == t[nk-1] falls into the closed last span), or -1 when x lies outside
// [t[0], t[nk-1]] or is NaN.  Descends over power-of-two strides: seven probes cover 72 knots, no
// data-dependent loop count.
template <typename T>
__host__ __device__ __forceinline__ int locate_span(const T* __restrict__ t, int nk, T x) {
    if (!(x >= t[0] && x <= t[nk - 1])) return -1;
    int m = 0;
#pragma unroll
    for (int stride = 64; stride > 0; stride >>= 1) {
        const int probe = m + stride;
        if (probe <= nk - 2 && t[probe] <= x) m = probe;
    }
    return m;
}

// b / den with the "0 / 0 = 0" rule of the recurrence folded in by the caller.  IEEE division for
// double; for float the 2-ulp fast division (the float kernels are compared at 1e-5, the double
// ones at 1e-12).
template <typename T> __host__ __device__ __forceinline__ T quotient(T b, T den) { return b / den; }
template <> __host__ __device__ __forceinline__ float quotient<float>(float b, float den) {
#ifdef __CUDA_ARCH__
    return __fdividef(b, den);
#else
    return b / den;
#endif
}

// Values (and, with DERIV, x-derivatives) of the K + 1 B-splines of degree K that can be non-zero
// on span m: window slot j stands for basis index m - K + j.
//
// Degree by degree, the functions of degree d - 1 are first divided by the knot difference their
// support spans,
//        q_j = B_{m-d+1+j, d-1} / (t_{m+1+j} - t_{m+1+j-d}),        j = 0 .. d-1   (0 where the knots coincide)
// which is the one quantity both terms of the Cox-de Boor step share:
//        B_{m-d+j, d} = (x - t_{m-d+j}) q_{j-1} + (t_{m+1+j} - x) q_j.
// At the last degree the same q give the derivative for free:
//        d/dx B_{m-K+j, K} = K (q_{j-1} - q_j).
// Knot reads beyond either end of the vector are clamped; they only reach slots whose basis
// index lies outside [0, R), which the caller drops.
template <int K, typename T, bool DERIV>
__host__ __device__ __forceinline__ void window_values(const T* __restrict__ t, int nk, int m, T x,
                                              T (&val)[K + 1], T (&der)[K + 1]) {
    T kn[2 * K];                        // kn[K - 1 + e] = t[m + e],  e = 1-K .. K
#pragma unroll
    for (int e = 0; e < 2 * K; ++e) {
        int at = m - K + 1 + e;
        at = at < 0 ? 0 : (at > nk - 1 ? nk - 1 : at);
        kn[e] = t[at];
    }
    T b[K + 1];
    b[0] = T(1);
#pragma unroll
    for (int j = 1; j <= K; ++j) b[j] = T(0);
#pragma unroll
    for (int d = 1; d <= K; ++d) {
        T q[K + 1];
#pragma unroll
        for (int j = 0; j < d; ++j) {
            const T width = kn[K + j] - kn[K + j - d];
            q[j] = (width != T(0)) ? quotient<T>(b[j], width) : T(0);
        }
        if (DERIV && d == K) {
#pragma unroll
            for (int j = 0; j <= K; ++j)
                der[j] = T(K) * ((j > 0 ? q[j - 1] : T(0)) - (j < K ? q[j] : T(0)));
        }
#pragma unroll
        for (int j = d; j >= 0; --j) {
            const T rising = (j > 0) ? (x - kn[K - 1 - d + j]) * q[j - 1] : T(0);
            const T falling = (j < d) ? (kn[K + j] - x) * q[j] : T(0);
            b[j] = rising + falling;
        }
    }
#pragma unroll
    for (int j = 0; j <= K; ++j) val[j] = b[j];
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
