// Refit of the spline coefficients after the knots of a layer moved (the second half of
// update_grid; reference: ReferenceKANLayer.update_grid + curve2coeff,
// spline_kan/reference_backend.py:218-265, 442-493, which samples every old curve at every input,
// materialises them as [O, B, I] and solves one least-squares system per input feature in a
// Python loop on the CPU).
//
// The least-squares fit of  sum_r c_new[o,i,r] B_new,r(x)  to the old curve
// sum_s c_old[o,i,s] B_old,s(x)  at the samples x[n,i] has the normal equations
//        G_i c_new[o,i,:] = M_i c_old[o,i,:],
//        G_i[r,r'] = sum_n B_new,r(x[n,i]) B_new,r'(x[n,i]),   M_i[r,s] = sum_n B_new,r(x[n,i]) B_old,s(x[n,i]),
// so the sampled curves are never needed: two [R, R] moment matrices per input feature hold
// everything, the outputs only enter through c_old, and  c_new[o,i,:] = (G_i^-1 M_i) c_old[o,i,:].
//
//   refit_moments_kernel   one block per feature: both windows of k+1 values per sample (float64),
//                          (k+1)^2 products into each matrix in shared memory
//   refit_solve_kernel     one block per feature: Cholesky of G_i, X_i = G_i^-1 M_i in place; a
//                          pivot below 1e-10 of the largest diagonal entry marks the feature as not
//                          safely positive definite (info != 0) and the host refits it by the
//                          minimum-norm path instead
#include "kan_device.cuh"
#include "kan_internal.h"

namespace kanb200 {

namespace {

constexpr int RF_THREADS = 256;
constexpr int RF_MAX_R = 72;

template <typename T, int K>
__global__ void __launch_bounds__(RF_THREADS)
refit_moments_kernel(const T* __restrict__ x, const T* __restrict__ grid_old, const T* __restrict__ grid_new,
                     double* __restrict__ Gm, double* __restrict__ Mm, int64_t N, int I, int R) {
    extern __shared__ double sm[];
    const int nk = R + K + 1;
    double* Gs = sm;                         // [R][R]
    double* Ms = Gs + R * R;                 // [R][R]
    double* t_old = Ms + R * R;              // [nk]
    double* t_new = t_old + nk;              // [nk]
    const int i = blockIdx.x, tid = threadIdx.x;
    for (int e = tid; e < 2 * R * R; e += RF_THREADS) sm[e] = 0.0;
    for (int e = tid; e < nk; e += RF_THREADS) {
        t_old[e] = (double)grid_old[(size_t)i * nk + e];
        t_new[e] = (double)grid_new[(size_t)i * nk + e];
    }
    __syncthreads();
    for (int64_t n = tid; n < N; n += RF_THREADS) {
        const double xv = (double)x[(size_t)n * I + i];
        const int mn = locate_span(t_new, nk, xv);
        if (mn < 0) continue;                               // outside the new knots: an all-zero row
        double vn[K + 1], vo[K + 1], unused[K + 1];
        window_values<K, double, false>(t_new, nk, mn, xv, vn, unused);
        const int mo = locate_span(t_old, nk, xv);
        if (mo >= 0) window_values<K, double, false>(t_old, nk, mo, xv, vo, unused);
#pragma unroll
        for (int a = 0; a <= K; ++a) {
            const int r = mn - K + a;
            if (r < 0 || r >= R) continue;
#pragma unroll
            for (int b = 0; b <= K; ++b) {
                const int r2 = mn - K + b;
                if (r2 >= 0 && r2 < R) atomicAdd(&Gs[r * R + r2], vn[a] * vn[b]);
                if (mo >= 0) {
                    const int s = mo - K + b;
                    if (s >= 0 && s < R) atomicAdd(&Ms[r * R + s], vn[a] * vo[b]);
                }
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < R * R; e += RF_THREADS) {
        Gm[(size_t)i * R * R + e] = Gs[e];
        Mm[(size_t)i * R * R + e] = Ms[e];
    }
}

// In place: G_i -> its Cholesky factor (lower triangle), M_i -> X_i = G_i^-1 M_i.
__global__ void __launch_bounds__(128)
refit_solve_kernel(double* __restrict__ Gm, double* __restrict__ Mm, int* __restrict__ info, int R) {
    extern __shared__ double sm[];
    double* L = sm;                          // [R][R + 1]
    double* X = L + R * (R + 1);             // [R][R + 1]
    __shared__ double max_diag;
    __shared__ int bad;
    const int i = blockIdx.x, tid = threadIdx.x, ld = R + 1;
    for (int e = tid; e < R * R; e += blockDim.x) {
        const int r = e / R, c = e - r * R;
        L[r * ld + c] = Gm[(size_t)i * R * R + e];
        X[r * ld + c] = Mm[(size_t)i * R * R + e];
    }
    if (tid == 0) bad = 0;
    __syncthreads();
    if (tid == 0) {
        double m = 0.0;
        for (int r = 0; r < R; ++r) m = fmax(m, L[r * ld + r]);
        max_diag = m;
    }
    __syncthreads();
    const double floor_pivot = 1e-10 * max_diag;
    for (int j = 0; j < R; ++j) {
        if (tid == 0) {
            double d = L[j * ld + j];
            for (int q = 0; q < j; ++q) d -= L[j * ld + q] * L[j * ld + q];
            if (!(d > floor_pivot)) {
                bad = j + 1;
                d = 1.0;
            }
            L[j * ld + j] = sqrt(d);
        }
        __syncthreads();
        if (bad) break;
        const double inv = 1.0 / L[j * ld + j];
        for (int r = j + 1 + tid; r < R; r += blockDim.x) {
            double v = L[r * ld + j];
            for (int q = 0; q < j; ++q) v -= L[r * ld + q] * L[j * ld + q];
            L[r * ld + j] = v * inv;
        }
        __syncthreads();
    }
    if (tid == 0) info[i] = (max_diag > 0.0) ? bad : 1;
    if (bad || !(max_diag > 0.0)) return;
    // one right-hand side (a column of M_i) per thread: L z = m, then L^T x = z
    for (int c = tid; c < R; c += blockDim.x) {
        for (int r = 0; r < R; ++r) {
            double v = X[r * ld + c];
            for (int q = 0; q < r; ++q) v -= L[r * ld + q] * X[q * ld + c];
            X[r * ld + c] = v / L[r * ld + r];
        }
        for (int r = R - 1; r >= 0; --r) {
            double v = X[r * ld + c];
            for (int q = r + 1; q < R; ++q) v -= L[q * ld + r] * X[q * ld + c];
            X[r * ld + c] = v / L[r * ld + r];
        }
    }
    __syncthreads();
    for (int e = tid; e < R * R; e += blockDim.x) {
        const int r = e / R, c = e - r * R;
        Mm[(size_t)i * R * R + e] = X[r * ld + c];
    }
}

template <typename T>
cudaError_t launch_moments(const T* x, const T* grid_old, const T* grid_new, double* Gm, double* Mm, int64_t N,
                           int I, int R, int k, cudaStream_t st) {
    const int nk = R + k + 1;
    const size_t smem = ((size_t)2 * R * R + 2 * nk) * sizeof(double);
    cudaError_t e = cudaSuccess;
#define KAN_RF(KK)                                                                                              \
    do {                                                                                                       \
        if (smem > 48 * 1024)                                                                                  \
            e = cudaFuncSetAttribute(refit_moments_kernel<T, KK>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                     (int)smem);                                                               \
        if (e == cudaSuccess)                                                                                  \
            refit_moments_kernel<T, KK><<<I, RF_THREADS, smem, st>>>(x, grid_old, grid_new, Gm, Mm, N, I, R);  \
    } while (0)
    if (k == 1) KAN_RF(1);
    else if (k == 2) KAN_RF(2);
    else KAN_RF(3);
#undef KAN_RF
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

template <typename T>
cudaError_t refit_moments(const T* x, const T* grid_old, const T* grid_new, double* Gm, double* Mm, int64_t N, int I,
                          int R, int k, cudaStream_t st) {
    if (R < 1 || R > RF_MAX_R) return cudaErrorInvalidValue;
    return launch_moments<T>(x, grid_old, grid_new, Gm, Mm, N, I, R, k, st);
}

cudaError_t refit_solve(double* Gm, double* Mm, int* info, int I, int R, cudaStream_t st) {
    if (R < 1 || R > RF_MAX_R) return cudaErrorInvalidValue;
    const size_t smem = (size_t)2 * R * (R + 1) * sizeof(double);
    cudaError_t e = cudaSuccess;
    if (smem > 48 * 1024)
        e = cudaFuncSetAttribute(refit_solve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    refit_solve_kernel<<<I, 128, smem, st>>>(Gm, Mm, info, R);
    return cudaGetLastError();
}

template cudaError_t refit_moments<float>(const float*, const float*, const float*, double*, double*, int64_t, int,
                                          int, int, cudaStream_t);
template cudaError_t refit_moments<double>(const double*, const double*, const double*, double*, double*, int64_t,
                                           int, int, int, cudaStream_t);

}  // namespace kanb200
