// Activation-regulariser statistic and its gradients, without ever storing
// phi[n,o,i] = s[n,i] bw[o,i] + sum_r H[n,i,r] W[o,i,r]:
//
//   forward   a[o,i]   = (1/N) sum_n |phi|
//   backward  g        = ga[o,i] sign(phi) / N        (sign(0) = 0)
//             dbw[o,i] = sum_n g s      dW[o,i,r] = sum_n g H[n,i,r]
//             ds[n,i]  = sum_o g bw     dH[n,i,r] = sum_o g W[o,i,r]
//
// Every kernel exists in two forms: from the materialised basis H [N,I,R] and base values s [N,I]
// (the operator surface of the reference, csrc/kan_reg_cuda.cu) and -- template parameter K > 0 --
// straight from the layer input x, where a block rebuilds the rows of H it needs in shared memory
// (parameter kernels) or registers (input kernel), the input kernel contracts dH with dB/dx on the
// spot, and neither H nor dH ever exists in memory.
//
// Bound by the FP32/FP64 FMA pipe (N O I (R+1) FMAs against N I (R+1) + O I (R+1)
// input elements).  Sums over samples are split across blocks; each split
// writes its own slab in the caller's workspace and a second kernel adds the
// slabs in a fixed order -- no atomics, bit-reproducible results.
#include <type_traits>

#include "kan_device.cuh"
#include "kan_internal.h"

namespace kanb200 {

namespace {

template <typename T>
__device__ __forceinline__ T sign_t(T v) { return T((v > T(0)) - (v < T(0))); }

constexpr int EA_TI = 4, EA_THREADS = 128;

// Reads CNT consecutive values from a 16-byte aligned shared-memory row with 16-byte loads.
template <typename T, int CNT>
__device__ __forceinline__ void load_row16(const T* __restrict__ p, T (&out)[CNT]) {
    constexpr int PER = 16 / sizeof(T);
    static_assert(CNT % PER == 0, "row length must be a multiple of 16 bytes");
    struct __align__(16) Pack { T v[PER]; };
#pragma unroll
    for (int q = 0; q < CNT / PER; ++q) {
        const Pack pk = reinterpret_cast<const Pack*>(p)[q];
#pragma unroll
        for (int e = 0; e < PER; ++e) out[q * PER + e] = pk.v[e];
    }
}

// Thread = OPT outputs x one feature, W rows in registers; loops over the
// samples of its split with H / s tiles staged in shared memory.
// K = 0: H and s are read from memory.  K = 1..3: H rows are evaluated from x on the knots `grid`
// (spline order K), and the base value is s[n,i] when s is given, silu(x) otherwise.
template <typename T, int RMAX, int OPT, int TNS, bool GRAD, int K>
__global__ void __launch_bounds__(EA_THREADS)
edge_param_kernel(const T* __restrict__ s, const T* __restrict__ H, const T* __restrict__ bw,
                  const T* __restrict__ W, const T* __restrict__ ga,
                  T* __restrict__ part_a, T* __restrict__ part_dbw, T* __restrict__ part_dW,
                  int64_t N, int I, int O, int R, int64_t n_per_split,
                  const T* __restrict__ x, const T* __restrict__ grid) {
    constexpr int TO = 32 * OPT;
    __shared__ __align__(16) T Hs[TNS][EA_TI][RMAX];
    __shared__ T ss[TNS][EA_TI];
    __shared__ T knots[K > 0 ? EA_TI : 1][K > 0 ? kMaxKnots : 1];
    const int nk = R + K + 1;
    const int tid = threadIdx.x;
    const int lane_o = tid & 31, ti = tid >> 5;
    const int o0 = blockIdx.x * TO, i0 = blockIdx.y * EA_TI;
    const int i = i0 + ti;
    const int64_t nb = (int64_t)blockIdx.z * n_per_split;
    const int64_t ne = (nb + n_per_split < N) ? nb + n_per_split : N;
    const T invN = T(1) / T(N);
    const bool has_base = (bw != nullptr);

    T w[OPT][RMAX], bwv[OPT], gav[OPT];
    T acc_a[OPT], acc_b[OPT];
    T dw[GRAD ? OPT : 1][GRAD ? RMAX : 1];
#pragma unroll
    for (int u = 0; u < OPT; ++u) {
        const int o = o0 + lane_o + 32 * u;
        const bool ok = (o < O) && (i < I);
        const size_t oi = ok ? (size_t)o * I + i : 0;
#pragma unroll
        for (int r = 0; r < RMAX; ++r) w[u][r] = (ok && r < R) ? W[oi * R + r] : T(0);
        bwv[u] = (ok && has_base) ? bw[oi] : T(0);
        gav[u] = (GRAD && ok) ? ga[oi] * invN : T(0);
        acc_a[u] = T(0);
        acc_b[u] = T(0);
        if (GRAD) {
#pragma unroll
            for (int r = 0; r < RMAX; ++r) dw[u][r] = T(0);
        }
    }

    if constexpr (K > 0) {
        for (int e = tid; e < EA_TI * nk; e += EA_THREADS) {
            const int ii = e / nk, q = e - ii * nk;
            knots[ii][q] = (i0 + ii < I) ? grid[(size_t)(i0 + ii) * nk + q] : T(0);
        }
    }

    for (int64_t nt = nb; nt < ne; nt += TNS) {
        __syncthreads();
        if constexpr (K == 0) {
            for (int e = tid; e < TNS * EA_TI * RMAX; e += EA_THREADS) {
                const int n = e / (EA_TI * RMAX);
                const int rem = e - n * (EA_TI * RMAX);
                const int ii = rem / RMAX, r = rem - ii * RMAX;
                T v = T(0);
                if (nt + n < ne && i0 + ii < I && r < R) v = H[((size_t)(nt + n) * I + i0 + ii) * R + r];
                Hs[n][ii][r] = v;
            }
            for (int e = tid; e < TNS * EA_TI; e += EA_THREADS) {
                const int n = e / EA_TI, ii = e - n * EA_TI;
                ss[n][ii] = (has_base && nt + n < ne && i0 + ii < I) ? s[(size_t)(nt + n) * I + i0 + ii] : T(0);
            }
        } else {
            // one (sample, feature) pair per thread and round: its dense basis row and base value
            for (int e = tid; e < TNS * EA_TI; e += EA_THREADS) {
                const int n = e / EA_TI, ii = e - n * EA_TI;
                T* row = &Hs[n][ii][0];
#pragma unroll
                for (int r = 0; r < RMAX; ++r) row[r] = T(0);
                T sv = T(0);
                if (nt + n < ne && i0 + ii < I) {
                    const size_t at = (size_t)(nt + n) * I + i0 + ii;
                    const T xv = x[at];
                    const int m = locate_span(&knots[ii][0], nk, xv);
                    if (m >= 0) {
                        T v[K + 1], d[K + 1];
                        window_values<K, T, false>(&knots[ii][0], nk, m, xv, v, d);
#pragma unroll
                        for (int j = 0; j <= K; ++j) {
                            const int r = m - K + j;
                            if (r >= 0 && r < R) row[r] = v[j];
                        }
                    }
                    if (has_base) sv = s ? s[at] : silu_t<T>(xv);
                }
                ss[n][ii] = sv;
            }
        }
        __syncthreads();
        const int lim = (int)((ne - nt < TNS) ? (ne - nt) : TNS);
        for (int n = 0; n < lim; ++n) {
            const T sv = ss[n][ti];
            T hrow[RMAX];
            load_row16<T, RMAX>(&Hs[n][ti][0], hrow);
            T phi[OPT];
#pragma unroll
            for (int u = 0; u < OPT; ++u) phi[u] = sv * bwv[u];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
#pragma unroll
                for (int u = 0; u < OPT; ++u) phi[u] += hrow[r] * w[u][r];
            }
            if (!GRAD) {
#pragma unroll
                for (int u = 0; u < OPT; ++u) acc_a[u] += fabs(phi[u]);
            } else {
                T g[OPT];
#pragma unroll
                for (int u = 0; u < OPT; ++u) {
                    g[u] = gav[u] * sign_t<T>(phi[u]);
                    acc_b[u] += g[u] * sv;
                }
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
#pragma unroll
                    for (int u = 0; u < OPT; ++u) dw[u][r] += g[u] * hrow[r];
                }
            }
        }
    }
    if (i < I) {
#pragma unroll
        for (int u = 0; u < OPT; ++u) {
            const int o = o0 + lane_o + 32 * u;
            if (o >= O) continue;
            const size_t oi = (size_t)blockIdx.z * O * I + (size_t)o * I + i;
            if (!GRAD) {
                part_a[oi] = acc_a[u];
            } else {
                if (part_dbw) part_dbw[oi] = acc_b[u];
                if (part_dW) {
#pragma unroll
                    for (int r = 0; r < RMAX; ++r)
                        if (r < R) part_dW[oi * R + r] = dw[u][r];
                }
            }
        }
    }
}

template <typename T>
__global__ void sum_slabs_kernel(const T* __restrict__ part, T* __restrict__ out, int64_t elems,
                                 int splits, T scale) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < elems;
         e += (int64_t)gridDim.x * blockDim.x) {
        T v = T(0);
        for (int s = 0; s < splits; ++s) v += part[(size_t)s * elems + e];
        out[e] = v * scale;
    }
}

// ga/N with the sign of phi (0 where phi == 0): the factor g of the backward formulas.
template <typename T>
__device__ __forceinline__ T signed_weight(T c, T phi) {
    return phi > T(0) ? c : (phi < T(0) ? -c : T(0));
}
template <>
__device__ __forceinline__ float signed_weight<float>(float c, float phi) {
    // c with its sign flipped where phi is negative
    const float flipped = __int_as_float(__float_as_int(c) ^ (__float_as_int(phi) & 0x80000000));
    return phi == 0.0f ? 0.0f : flipped;
}

// Thread = NPT samples x one feature: their H rows and dH accumulators in registers; loops over
// tiles of outputs staged in shared memory (a weight row is read once per NPT samples).
constexpr int EB_TI = 4, EB_TN = 32, EB_THREADS = 128;

// K = 0: H rows are read, ds and dH are written.  K = 1..3: the rows are evaluated from x, dH is
// contracted with dB/dx in registers and the kernel writes the input gradient
//     gx[n,i] = sum_r dH[n,i,r] dB_r/dx (x[n,i])  ( + ds[n,i] silu'(x[n,i]) when s is NULL )
// and, when the caller supplied its own base values s, ds [N,I] for them.
template <typename T, int RMAX, int TOC, int NPT, int K>
__global__ void __launch_bounds__(EB_THREADS)
edge_input_kernel(const T* __restrict__ s, const T* __restrict__ H, const T* __restrict__ bw,
                  const T* __restrict__ W, const T* __restrict__ ga,
                  T* __restrict__ ds, T* __restrict__ dH,
                  int64_t N, int I, int O, int R,
                  const T* __restrict__ x, const T* __restrict__ grid, T* __restrict__ gx) {
    constexpr int WROW = RMAX + 16 / sizeof(T);   // 16-byte aligned rows: [RMAX] = bw, [RMAX+1] = ga/N
    __shared__ __align__(16) T Ws[TOC][EB_TI][WROW];
    __shared__ T knots[K > 0 ? EB_TI : 1][K > 0 ? kMaxKnots : 1];
    const int nk = R + K + 1;
    const int tid = threadIdx.x;
    const int ti = tid & (EB_TI - 1), tn = tid / EB_TI;
    const int i0 = blockIdx.y * EB_TI;
    const int i = i0 + ti;
    const int64_t nbase = (int64_t)blockIdx.x * (EB_TN * NPT) + tn;
    const bool has_base = (bw != nullptr);
    const T invN = T(1) / T(N);

    T h[NPT][RMAX], dh[NPT][RMAX], sv[NPT], dsv[NPT];
    T der[K > 0 ? NPT : 1][K + 1], xq[K > 0 ? NPT : 1];
    int first[K > 0 ? NPT : 1];          // basis index of window slot 0 (may be negative)
    bool live[NPT];
    if constexpr (K > 0) {
        for (int e = tid; e < EB_TI * nk; e += EB_THREADS) {
            const int ii = e / nk, q = e - ii * nk;
            knots[ii][q] = (i0 + ii < I) ? grid[(size_t)(i0 + ii) * nk + q] : T(0);
        }
        __syncthreads();
    }
#pragma unroll
    for (int q = 0; q < NPT; ++q) {
        const int64_t n = nbase + (int64_t)q * EB_TN;
        live[q] = (i < I) && (n < N);
        dsv[q] = T(0);
#pragma unroll
        for (int r = 0; r < RMAX; ++r) dh[q][r] = T(0);
        if constexpr (K == 0) {
#pragma unroll
            for (int r = 0; r < RMAX; ++r) h[q][r] = (live[q] && r < R) ? H[((size_t)n * I + i) * R + r] : T(0);
            sv[q] = (live[q] && has_base) ? s[(size_t)n * I + i] : T(0);
        } else {
#pragma unroll
            for (int r = 0; r < RMAX; ++r) h[q][r] = T(0);
#pragma unroll
            for (int j = 0; j <= K; ++j) der[q][j] = T(0);
            sv[q] = T(0);
            xq[q] = T(0);
            first[q] = 0;
            if (live[q]) {
                const T xv = x[(size_t)n * I + i];
                xq[q] = xv;
                const int m = locate_span(&knots[ti][0], nk, xv);
                if (m >= 0) {
                    T v[K + 1];
                    window_values<K, T, true>(&knots[ti][0], nk, m, xv, v, der[q]);
                    first[q] = m - K;
                    // registers cannot be indexed by m: every slot picks its value by comparison
#pragma unroll
                    for (int r = 0; r < RMAX; ++r) {
#pragma unroll
                        for (int j = 0; j <= K; ++j) h[q][r] = (r == m - K + j && r < R) ? v[j] : h[q][r];
                    }
                }
                if (has_base) sv[q] = s ? s[(size_t)n * I + i] : silu_t<T>(xv);
            }
        }
    }

    for (int oc = 0; oc < O; oc += TOC) {
        __syncthreads();
        for (int e = tid; e < TOC * EB_TI * (RMAX + 2); e += EB_THREADS) {
            const int o = e / (EB_TI * (RMAX + 2));
            const int rem = e - o * (EB_TI * (RMAX + 2));
            const int ii = rem / (RMAX + 2), r = rem - ii * (RMAX + 2);
            // (the padding slots beyond RMAX + 1 are never read as data)
            T v = T(0);
            if (oc + o < O && i0 + ii < I) {
                const size_t oi = (size_t)(oc + o) * I + i0 + ii;
                if (r < RMAX) v = (r < R) ? W[oi * R + r] : T(0);
                else if (r == RMAX) v = has_base ? bw[oi] : T(0);
                else v = ga[oi] * invN;
            }
            Ws[o][ii][r] = v;
        }
        __syncthreads();
#pragma unroll 1
        for (int o = 0; o < TOC; ++o) {
            // narrow rows are copied to registers with 16-byte loads; wide ones are read in place
            constexpr int WREG = RMAX <= 16 ? WROW : 1;
            T wreg[WREG];
            if constexpr (RMAX <= 16) load_row16<T, WROW>(&Ws[o][ti][0], wreg);
            const T* wr = RMAX <= 16 ? wreg : &Ws[o][ti][0];
#pragma unroll
            for (int q = 0; q < NPT; ++q) {
                T phi = sv[q] * wr[RMAX];
#pragma unroll
                for (int r = 0; r < RMAX; ++r) phi += h[q][r] * wr[r];
                const T g = signed_weight<T>(wr[RMAX + 1], phi);
                dsv[q] += g * wr[RMAX];
#pragma unroll
                for (int r = 0; r < RMAX; ++r) dh[q][r] += g * wr[r];
            }
        }
    }
#pragma unroll
    for (int q = 0; q < NPT; ++q) {
        if (!live[q]) continue;
        const int64_t n = nbase + (int64_t)q * EB_TN;
        if (ds) ds[(size_t)n * I + i] = dsv[q];
        if constexpr (K == 0) {
            if (dH) {
#pragma unroll
                for (int r = 0; r < RMAX; ++r)
                    if (r < R) dH[((size_t)n * I + i) * R + r] = dh[q][r];
            }
        } else {
            if (gx) {
                T g = (has_base && !s) ? dsv[q] * silu_grad_t<T>(xq[q]) : T(0);
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    T d = T(0);
#pragma unroll
                    for (int j = 0; j <= K; ++j) d = (r == first[q] + j && r < R) ? der[q][j] : d;
                    g += dh[q][r] * d;
                }
                gx[(size_t)n * I + i] = g;
            }
        }
    }
}

struct EdgePlan {
    int rmax, opt, tns, to, splits;
    int64_t n_per_split;
};

// Resident blocks per SM of the parameter kernel that plan_edge would launch (asked from the
// runtime once per instantiation; a build-time estimate when no device can be asked).
template <typename T, bool GRAD>
int edge_param_blocks_per_sm(int rmax) {
    static int cached[4] = {0, 0, 0, 0};
    const int slot = rmax == 8 ? 0 : (rmax == 16 ? 1 : (rmax == 32 ? 2 : 3));
    if (cached[slot] > 0) return cached[slot];
    int n = 0;
    cudaError_t e;
    if (rmax == 8)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, edge_param_kernel<T, 8, 4, 32, GRAD, 0>, EA_THREADS, 0);
    else if (rmax == 16)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, edge_param_kernel<T, 16, 2, 32, GRAD, 0>, EA_THREADS, 0);
    else if (rmax == 32)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, edge_param_kernel<T, 32, 1, 8, GRAD, 0>, EA_THREADS, 0);
    else
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, edge_param_kernel<T, 72, 1, 8, GRAD, 0>, EA_THREADS, 0);
    if (e != cudaSuccess || n < 1) {
        cudaGetLastError();
        return GRAD ? 2 : 4;            // not cached: a later call with a device asks again
    }
    cached[slot] = n;
    return n;
}

inline int edge_sm_count() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            cached = n;
        else {
            cudaGetLastError();
            return 148;
        }
    }
    return cached;
}

// Split of the sample range: the number of blocks is brought close to a whole number of waves
// (resident blocks on the whole device), since a partly filled last wave costs a full one.
template <typename T, bool GRAD>
EdgePlan plan_edge(int64_t N, int I, int O, int R) {
    EdgePlan p;
    p.rmax = R <= 8 ? 8 : (R <= 16 ? 16 : (R <= 32 ? 32 : 72));
    p.opt = p.rmax <= 8 ? 4 : (p.rmax == 16 ? 2 : 1);
    p.tns = p.rmax >= 32 ? 8 : 32;
    p.to = 32 * p.opt;
    const int64_t bxy = (int64_t)((O + p.to - 1) / p.to) * ((I + EA_TI - 1) / EA_TI);
    const int64_t wave = (int64_t)edge_sm_count() * edge_param_blocks_per_sm<T, GRAD>(p.rmax);
    int64_t max_splits = (N + 127) / 128;
    if (max_splits > 64) max_splits = 64;
    if (max_splits < 1) max_splits = 1;
    int64_t best = 1;
    double best_eff = 0.0;
    for (int64_t sp = 1; sp <= max_splits; ++sp) {
        const int64_t blocks = bxy * sp;
        const int64_t waves = (blocks + wave - 1) / wave;
        // fraction of the occupied block slots that do work, discounted a little per extra slab
        const double eff = (double)blocks / (double)(waves * wave) - 0.004 * (double)(sp - 1);
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best = sp;
        }
        if (blocks >= 8 * wave) break;      // many waves: the tail no longer matters
    }
    p.n_per_split = (N + best - 1) / best;
    p.splits = (int)((N + p.n_per_split - 1) / p.n_per_split);
    if (p.splits < 1) p.splits = 1;
    return p;
}

// K = 0: from H / s.  K > 0: from x on the knots `grid`.
template <typename T, bool GRAD, int K>
cudaError_t launch_edge_param(const EdgePlan& p, const T* s, const T* H, const T* bw, const T* W, const T* ga,
                              T* pa, T* pdbw, T* pdW, int64_t N, int I, int O, int R, cudaStream_t st,
                              const T* x = nullptr, const T* grid = nullptr) {
    dim3 g((O + p.to - 1) / p.to, (I + EA_TI - 1) / EA_TI, p.splits);
#define KAN_EP(RM, OP, TN)                                                                              \
    edge_param_kernel<T, RM, OP, TN, GRAD, K><<<g, EA_THREADS, 0, st>>>(s, H, bw, W, ga, pa, pdbw, pdW, \
                                                                        N, I, O, R, p.n_per_split, x, grid)
    if (p.rmax == 8) KAN_EP(8, 4, 32);
    else if (p.rmax == 16) KAN_EP(16, 2, 32);
    else if (p.rmax == 32) KAN_EP(32, 1, 8);
    else KAN_EP(72, 1, 8);
#undef KAN_EP
    return cudaGetLastError();
}

template <typename T, int K>
cudaError_t launch_edge_input(const T* s, const T* H, const T* bw, const T* W, const T* ga, T* ds, T* dH,
                              int64_t N, int I, int O, int R, cudaStream_t st,
                              const T* x = nullptr, const T* grid = nullptr, T* gx = nullptr) {
    const int rmax = R <= 8 ? 8 : (R <= 16 ? 16 : (R <= 32 ? 32 : 72));
    const int npt = rmax == 8 ? 4 : (rmax == 16 ? 2 : 1);   // samples per thread
    dim3 g((unsigned)((N + EB_TN * npt - 1) / (EB_TN * npt)), (I + EB_TI - 1) / EB_TI);
    if (rmax == 8) edge_input_kernel<T, 8, 32, 4, K><<<g, EB_THREADS, 0, st>>>(s, H, bw, W, ga, ds, dH, N, I, O, R, x, grid, gx);
    else if (rmax == 16) edge_input_kernel<T, 16, 32, 2, K><<<g, EB_THREADS, 0, st>>>(s, H, bw, W, ga, ds, dH, N, I, O, R, x, grid, gx);
    else if (rmax == 32) edge_input_kernel<T, 32, 16, 1, K><<<g, EB_THREADS, 0, st>>>(s, H, bw, W, ga, ds, dH, N, I, O, R, x, grid, gx);
    else edge_input_kernel<T, 72, 8, 1, K><<<g, EB_THREADS, 0, st>>>(s, H, bw, W, ga, ds, dH, N, I, O, R, x, grid, gx);
    return cudaGetLastError();
}

#define KAN_EDGE_K(Kval, ...)                                      \
    switch (Kval) {                                                \
        case 1: { constexpr int KK = 1; __VA_ARGS__; break; }      \
        case 2: { constexpr int KK = 2; __VA_ARGS__; break; }      \
        default: { constexpr int KK = 3; __VA_ARGS__; break; }     \
    }

inline int grid_1d(int64_t work, int threads, int cap = 148 * 32) {
    int64_t b = (work + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > cap) b = cap;
    return (int)b;
}

// ---------------------------------------------------------------------------
// Narrow layers (at most 16 outputs, at most 8 basis functions), from x: ONE kernel for the
// statistic (GRAD = false) or for all of its gradients (GRAD = true).
// ---------------------------------------------------------------------------
// The kernels above tile 32 outputs per weight tile and the tensor-core ones 128, so a layer with a
// handful of outputs (a classifier head: 256 -> 10) pays for outputs it does not have.  Here a block
// owns ONE feature and a range of samples; a thread walks samples of that range, builds the dense
// row A[0..7] of the feature's basis (k+1 non-zeros) and keeps one accumulator per (output, slot) in
// registers; the feature's weights sit in shared memory and are read as broadcasts.  Outputs are
// processed OT at a time (the samples are re-read per pass; the last pass is predicated).  Per-split
// slabs, summed in fixed order: no atomics.  Measured, 8192 rows, statistic / all gradients in us:
// 256 -> 10: 68 / 172 (tensor-core kernels 69 / 283, the 32-output FMA kernels 145 / 580), 256 -> 4:
// 49 / 105, 64 -> 16: 29 / 68 (37 / 110); 65536 rows, 64 -> 1: 90 / 195 (101 / 496).
constexpr int EN_THREADS = 128, EN_R = 8;            // EN_R: slots per feature of the edge kernels (R <= 8)
constexpr int kNarrowMaxO = 16;

// RM = slots kept per feature (8 or 16).  LAYER = false: the edge statistic (g = sign(phi) ga / N).
// LAYER = true: the backward of the layer itself, y = sum_i phi: g = dY[n, o] (passed as `ga`, [N, O]),
// phi is not needed, and `W` are the raw coefficients that `scaler` (may be NULL) multiplies.
template <typename T, int K, int OT, bool GRAD, int RM = EN_R, bool LAYER = false>
__global__ void __launch_bounds__(EN_THREADS)
edge_narrow_kernel(const T* __restrict__ x, const T* __restrict__ s, const T* __restrict__ grid,
                   const T* __restrict__ bw, const T* __restrict__ W, const T* __restrict__ ga,
                   T* __restrict__ pa, T* __restrict__ pdW, T* __restrict__ pdbw, T* __restrict__ gx,
                   T* __restrict__ ds, int64_t N, int I, int O, int R, int64_t rows_per_split,
                   const T* __restrict__ scaler = nullptr) {
    __shared__ T knots[kMaxKnots];
    constexpr int WROW = RM + 4;                       // rows start on 16-byte boundaries
    __shared__ __align__(16) T Ws[OT][WROW];             // [r < 8] weights, [8] base weight, [9] ga / N
    __shared__ T red[EN_THREADS / 32][OT * (RM + 1)];
    const int i = blockIdx.x, split = blockIdx.y, tid = threadIdx.x;
    const int nk = R + K + 1;
    const bool has_base = bw != nullptr;
    const T invN = T(1) / T(N);
    const int64_t n_begin = (int64_t)split * rows_per_split;
    const int64_t n_end = n_begin + rows_per_split < N ? n_begin + rows_per_split : N;
    for (int e = tid; e < nk; e += EN_THREADS) knots[e] = grid[(size_t)i * nk + e];
    const size_t oi_all = (size_t)O * I;

    for (int o0 = 0; o0 < O; o0 += OT) {
        __syncthreads();
        for (int e = tid; e < OT * WROW; e += EN_THREADS) {
            const int o = e / WROW, r = e - o * WROW;
            T v = T(0);
            if (o0 + o < O) {
                const size_t oi = (size_t)(o0 + o) * I + i;
                if (r < RM) v = r < R ? W[oi * R + r] * ((LAYER && scaler) ? scaler[oi] : T(1)) : T(0);
                else if (r == RM) v = has_base ? bw[oi] : T(0);
                else if (r == RM + 1) v = (GRAD && !LAYER && ga) ? ga[oi] * invN : T(0);
            }
            Ws[o][r] = v;
        }
        __syncthreads();
        T acc[OT][GRAD ? RM + 1 : 1];
#pragma unroll
        for (int o = 0; o < OT; ++o)
#pragma unroll
            for (int r = 0; r < (GRAD ? RM + 1 : 1); ++r) acc[o][r] = T(0);

        // the next sample's input (and base value) is loaded while this one is processed
        T x_next = n_begin + tid < n_end ? x[(size_t)(n_begin + tid) * I + i] : T(0);
        T s_next = (s && has_base && n_begin + tid < n_end) ? s[(size_t)(n_begin + tid) * I + i] : T(0);
        for (int64_t n = n_begin + tid; n < n_end; n += EN_THREADS) {
            const T xv = x_next, s_given = s_next;
            if (n + EN_THREADS < n_end) {
                x_next = x[(size_t)(n + EN_THREADS) * I + i];
                if (s && has_base) s_next = s[(size_t)(n + EN_THREADS) * I + i];
            }
            T A[RM], dA[RM];
#pragma unroll
            for (int r = 0; r < RM; ++r) { A[r] = T(0); dA[r] = T(0); }
            const int m = locate_span(knots, nk, xv);
            if (m >= 0) {
                T v[K + 1], d[K + 1];
                window_values<K, T, true>(knots, nk, m, xv, v, d);
                // registers cannot be indexed by m: every slot picks its value by comparison
#pragma unroll
                for (int r = 0; r < RM; ++r) {
#pragma unroll
                    for (int j = 0; j <= K; ++j) {
                        const bool hit = (r == m - K + j) && r < R;
                        A[r] = hit ? v[j] : A[r];
                        if (GRAD) dA[r] = hit ? d[j] : dA[r];
                    }
                }
            }
            const T sv = has_base ? (s ? s_given : silu_t<T>(xv)) : T(0);
            T g_basis = T(0), g_base = T(0);
#pragma unroll
            for (int o = 0; o < OT; ++o) {
                // the row of weights in 16-byte pieces (broadcast reads), used for phi and for dphi/dx
                T w[RM];
                {
                    using V = typename std::conditional<sizeof(T) == 4, float4, double2>::type;
                    constexpr int PER = 16 / sizeof(T);
                    const V* src = reinterpret_cast<const V*>(&Ws[o][0]);
#pragma unroll
                    for (int q = 0; q < RM / PER; ++q) {
                        const V v = src[q];
                        const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
                        for (int e = 0; e < PER; ++e) w[q * PER + e] = pv[e];
                    }
                }
                T phi = T(0);
                if (!LAYER) {
                    phi = Ws[o][RM] * sv;
#pragma unroll
                    for (int r = 0; r < RM; ++r) phi = fma(w[r], A[r], phi);
                }
                if (!GRAD) {
                    acc[o][0] += fabs(phi);
                } else {
                    const T g = LAYER ? (o0 + o < O ? ga[(size_t)n * O + o0 + o] : T(0))
                                      : signed_weight<T>(Ws[o][RM + 1], phi);
#pragma unroll
                    for (int r = 0; r < RM; ++r) acc[o][r] = fma(g, A[r], acc[o][r]);
                    acc[o][GRAD ? RM : 0] = fma(g, sv, acc[o][GRAD ? RM : 0]);
                    T dphi = T(0);
#pragma unroll
                    for (int r = 0; r < RM; ++r) dphi = fma(w[r], dA[r], dphi);
                    g_basis = fma(g, dphi, g_basis);
                    g_base = fma(g, Ws[o][RM], g_base);
                }
            }
            if (GRAD) {
                // outputs come in passes of OT: the first pass stores, the later ones add (same thread,
                // program order)
                if (gx) {
                    T v = g_basis;
                    if (has_base && !s) v = fma(g_base, silu_grad_t<T>(xv), v);
                    T* dst = gx + (size_t)n * I + i;
                    *dst = o0 == 0 ? v : *dst + v;
                }
                if (ds && s && has_base) {
                    T* dst = ds + (size_t)n * I + i;
                    *dst = o0 == 0 ? g_base : *dst + g_base;
                }
            }
        }

        // block sum of the accumulators: shuffles inside a warp, shared memory across the four warps
        constexpr int CNT = GRAD ? RM + 1 : 1;
#pragma unroll
        for (int o = 0; o < OT; ++o)
#pragma unroll
            for (int r = 0; r < CNT; ++r) {
                T v = acc[o][r];
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if ((tid & 31) == 0) red[tid >> 5][o * CNT + r] = v;
            }
        __syncthreads();
        for (int e = tid; e < OT * CNT; e += EN_THREADS) {
            const int o = e / CNT, r = e - o * CNT;
            if (o0 + o >= O) continue;
            T v = T(0);
            for (int w = 0; w < EN_THREADS / 32; ++w) v += red[w][e];
            const size_t oi = (size_t)(o0 + o) * I + i;
            if (!GRAD) {
                pa[(size_t)split * oi_all + oi] = v;
            } else if (r < RM) {
                if (pdW && r < R) pdW[((size_t)split * oi_all + oi) * R + r] = v;
            } else if (pdbw) {
                pdbw[(size_t)split * oi_all + oi] = v;
            }
        }
    }
}

// Layer forward for at most 16 outputs:  y[n, o] = sum_i ( bw[o,i] silu(x[n,i]) + sum_r W[o,i,r] scaler[o,i] B_r(x[n,i]) ).
// A block owns 64 samples; its 128 threads are 64 samples x 2 halves that take alternate chunks of
// eight features (knots and effective weights of a chunk staged in shared memory); a thread
// evaluates the k+1 non-zero basis values of its sample and gathers the matching coefficients.
constexpr int NF_FC = 8, NF_ROWS = 64;
template <typename T, int K, int OT>
__global__ void __launch_bounds__(EN_THREADS)
narrow_layer_forward_kernel(const T* __restrict__ x, const T* __restrict__ grid, const T* __restrict__ bw,
                            const T* __restrict__ sw, const T* __restrict__ scaler, T* __restrict__ y, int64_t N, int I,
                            int O, int R) {
    constexpr int RW = 20;                                   // R + 1 <= 17 values per (feature, output)
    __shared__ T knots[2][NF_FC][kMaxKnots];
    __shared__ T Ws[2][NF_FC][OT][RW];
    __shared__ T ysum[NF_ROWS][OT + 1];
    const int tid = threadIdx.x, half = tid >> 6, nl = tid & (NF_ROWS - 1);
    const int nk = R + K + 1;
    const int64_t n = (int64_t)blockIdx.x * NF_ROWS + nl;
    const bool row_ok = n < N;
    const bool has_base = bw != nullptr;
    const int n_chunks = (I + NF_FC - 1) / NF_FC;
    for (int o0 = 0; o0 < O; o0 += OT) {
        T acc[OT];
#pragma unroll
        for (int o = 0; o < OT; ++o) acc[o] = T(0);
        // both halves walk ceil(n_chunks / 2) rounds together (block barriers inside)
        for (int c0 = 0; c0 < n_chunks; c0 += 2) {
            __syncthreads();
            for (int e = tid; e < 2 * NF_FC * nk; e += EN_THREADS) {
                const int h = e / (NF_FC * nk), rem = e - h * (NF_FC * nk);
                const int fi = rem / nk, q = rem - fi * nk;
                const int i = (c0 + h) * NF_FC + fi;
                knots[h][fi][q] = i < I ? grid[(size_t)i * nk + q] : T(0);
            }
            for (int e = tid; e < 2 * NF_FC * OT * (R + 1); e += EN_THREADS) {
                const int h = e / (NF_FC * OT * (R + 1));
                int rem = e - h * (NF_FC * OT * (R + 1));
                const int fi = rem / (OT * (R + 1));
                rem -= fi * (OT * (R + 1));
                const int o = rem / (R + 1), r = rem - o * (R + 1);
                const int i = (c0 + h) * NF_FC + fi;
                T v = T(0);
                if (i < I && o0 + o < O) {
                    const size_t oi = (size_t)(o0 + o) * I + i;
                    if (r < R) v = sw[oi * R + r] * (scaler ? scaler[oi] : T(1));
                    else v = has_base ? bw[oi] : T(0);
                }
                Ws[h][fi][o][r] = v;
            }
            __syncthreads();
            const int i_first = (c0 + half) * NF_FC;
            if (row_ok && i_first < I) {
#pragma unroll 1
                for (int fi = 0; fi < NF_FC; ++fi) {
                    const int i = i_first + fi;
                    if (i >= I) break;
                    const T xv = x[(size_t)n * I + i];
                    const T sv = has_base ? silu_t<T>(xv) : T(0);
                    const int m = locate_span(&knots[half][fi][0], nk, xv);
                    T v[K + 1], unused[K + 1], w[K + 1];
                    if (m >= 0) window_values<K, T, false>(&knots[half][fi][0], nk, m, xv, v, unused);
                    const int first = window_in_range<K, T>(m, R, v, w);
#pragma unroll
                    for (int o = 0; o < OT; ++o) {
                        const T* wr = &Ws[half][fi][o][0];
                        T a = wr[R] * sv;
#pragma unroll
                        for (int j = 0; j <= K; ++j) a = fma(wr[first + j], w[j], a);
                        acc[o] += a;
                    }
                }
            }
        }
        // the two halves of a sample add up through shared memory
        __syncthreads();
        if (half == 1)
#pragma unroll
            for (int o = 0; o < OT; ++o) ysum[nl][o] = acc[o];
        __syncthreads();
        if (half == 0 && row_ok)
#pragma unroll
            for (int o = 0; o < OT; ++o)
                if (o0 + o < O) y[(size_t)n * O + o0 + o] = acc[o] + ysum[nl][o];
    }
}

// Parameter gradients of the narrow layer from the per-split slabs of edge_narrow_kernel<..., LAYER = true>:
// dW_eff = sum of the slabs; gsw = scaler dW_eff, gscaler = sum_r sw dW_eff, gbw = sum of its slabs.
template <typename T>
__global__ void narrow_layer_finalize_kernel(const T* __restrict__ pdW, const T* __restrict__ pdbw,
                                             const T* __restrict__ sw, const T* __restrict__ scaler,
                                             T* __restrict__ gsw, T* __restrict__ gscaler, T* __restrict__ gbw,
                                             int64_t oi_count, int R, int splits) {
    for (int64_t oi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; oi < oi_count;
         oi += (int64_t)gridDim.x * blockDim.x) {
        if (gsw || gscaler) {
            const T sc = scaler ? scaler[oi] : T(1);
            T gs = T(0);
            for (int r = 0; r < R; ++r) {
                T d = T(0);
                for (int sp = 0; sp < splits; ++sp) d += pdW[((size_t)sp * oi_count + oi) * R + r];
                if (gsw) gsw[oi * R + r] = sc * d;
                if (gscaler) gs += sw[oi * R + r] * d;
            }
            if (gscaler) gscaler[oi] = gs;
        }
        if (gbw) {
            T d = T(0);
            for (int sp = 0; sp < splits; ++sp) d += pdbw[(size_t)sp * oi_count + oi];
            gbw[oi] = d;
        }
    }
}

// Sample splits of the narrow kernels: about four blocks per SM, at least 256 samples per block.
inline int narrow_splits(int64_t N, int I) {
    int64_t want = (4 * (int64_t)edge_sm_count() + I - 1) / I;
    const int64_t most = (N + 255) / 256;
    if (want > most) want = most;
    if (want < 1) want = 1;
    if (want > 64) want = 64;
    return (int)want;
}
inline bool narrow_applies(int64_t N, int O, int R) { return O <= kNarrowMaxO && R <= EN_R && N >= 1; }

template <typename T, bool GRAD>
cudaError_t launch_edge_narrow(const T* x, const T* s, const T* grid, const T* bw, const T* W, const T* ga, T* pa,
                               T* pdW, T* pdbw, T* gx, T* ds, int64_t N, int I, int O, int R, int k, int splits,
                               cudaStream_t st) {
    const int64_t rows = (N + splits - 1) / splits;
    const dim3 blocks(I, splits);
    // outputs whose accumulators (nine each with gradients, one without) fit the register file:
    // float 16 (12 or 8 when the layer has no more: idle output slots cost their share of the work), double 4
    // with gradients and 8 without
    constexpr int OT_SMALL = sizeof(T) == 4 ? 8 : (GRAD ? 4 : 8);
    constexpr int OT_WIDE = sizeof(T) == 4 ? 16 : OT_SMALL;
    constexpr int OT_MID = sizeof(T) == 4 ? 12 : OT_SMALL;
    if (O > OT_SMALL && O <= OT_MID && OT_MID > OT_SMALL) {
        KAN_EDGE_K(k, (edge_narrow_kernel<T, KK, OT_MID, GRAD><<<blocks, EN_THREADS, 0, st>>>(
                          x, s, grid, bw, W, ga, pa, pdW, pdbw, gx, ds, N, I, O, R, rows)));
    } else if (O > OT_SMALL && OT_WIDE > OT_SMALL) {
        KAN_EDGE_K(k, (edge_narrow_kernel<T, KK, OT_WIDE, GRAD><<<blocks, EN_THREADS, 0, st>>>(
                          x, s, grid, bw, W, ga, pa, pdW, pdbw, gx, ds, N, I, O, R, rows)));
    } else {
        KAN_EDGE_K(k, (edge_narrow_kernel<T, KK, OT_SMALL, GRAD><<<blocks, EN_THREADS, 0, st>>>(
                          x, s, grid, bw, W, ga, pa, pdW, pdbw, gx, ds, N, I, O, R, rows)));
    }
    return cudaGetLastError();
}

}  // namespace

template <typename T>
size_t edge_workspace(int64_t N, int I, int O, int R, bool backward) {
    EdgePlan p = backward ? plan_edge<T, true>(N, I, O, R) : plan_edge<T, false>(N, I, O, R);
    const size_t oi = (size_t)O * I;
    int splits = p.splits;
    if (narrow_applies(N, O, R) && narrow_splits(N, I) > splits) splits = narrow_splits(N, I);   // from-x narrow kernels
    return (size_t)splits * oi * (backward ? (size_t)(R + 1) : 1) * sizeof(T);
}

template <typename T>
cudaError_t edge_abs_mean_fwd(const T* s, const T* H, const T* bw, const T* W, T* a,
                              int64_t N, int I, int O, int R, void* ws, size_t ws_bytes, cudaStream_t st) {
    EdgePlan p = plan_edge<T, false>(N, I, O, R);
    const size_t oi = (size_t)O * I;
    if (!ws || ws_bytes < (size_t)p.splits * oi * sizeof(T)) return cudaErrorMemoryAllocation;
    T* pa = reinterpret_cast<T*>(ws);
    cudaError_t e = launch_edge_param<T, false, 0>(p, s, H, bw, W, nullptr, pa, nullptr, nullptr, N, I, O, R, st);
    if (e != cudaSuccess) return e;
    sum_slabs_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pa, a, (int64_t)oi, p.splits, T(1) / T(N));
    return cudaGetLastError();
}

template <typename T>
cudaError_t edge_abs_mean_bwd(const T* ga, const T* s, const T* H, const T* bw, const T* W,
                              T* ds, T* dH, T* dbw, T* dW,
                              int64_t N, int I, int O, int R, void* ws, size_t ws_bytes, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    const size_t oi = (size_t)O * I;
    if (dbw || dW) {
        EdgePlan p = plan_edge<T, true>(N, I, O, R);
        if (!ws || ws_bytes < (size_t)p.splits * oi * (R + 1) * sizeof(T)) return cudaErrorMemoryAllocation;
        T* pdW = reinterpret_cast<T*>(ws);
        T* pdbw = pdW + (size_t)p.splits * oi * R;
        e = launch_edge_param<T, true, 0>(p, s, H, bw, W, ga, nullptr, (dbw && bw) ? pdbw : nullptr,
                                          dW ? pdW : nullptr, N, I, O, R, st);
        if (e != cudaSuccess) return e;
        if (dW) {
            sum_slabs_kernel<T><<<grid_1d((int64_t)oi * R, 256), 256, 0, st>>>(pdW, dW, (int64_t)oi * R, p.splits, T(1));
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        if (dbw && bw) {
            sum_slabs_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pdbw, dbw, (int64_t)oi, p.splits, T(1));
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
    }
    if ((ds && bw) || dH) e = launch_edge_input<T, 0>(s, H, bw, W, ga, (ds && bw) ? ds : nullptr, dH, N, I, O, R, st);
    return e;
}

// ---------------------------------------------------------------------------
// The same operators straight from the layer input x (spline order k, knots grid [I, R + k + 1])
// ---------------------------------------------------------------------------
template <typename T>
cudaError_t edge_abs_mean_x_fwd(const T* x, const T* s, const T* grid, const T* bw, const T* W, T* a,
                                int64_t N, int I, int O, int R, int k, void* ws, size_t ws_bytes, cudaStream_t st) {
    const size_t oi = (size_t)O * I;
    if (narrow_applies(N, O, R)) {
        const int splits = narrow_splits(N, I);
        if (!ws || ws_bytes < (size_t)splits * oi * sizeof(T)) return cudaErrorMemoryAllocation;
        T* pa = reinterpret_cast<T*>(ws);
        cudaError_t e = launch_edge_narrow<T, false>(x, s, grid, bw, W, nullptr, pa, nullptr, nullptr, nullptr,
                                                     nullptr, N, I, O, R, k, splits, st);
        if (e != cudaSuccess) return e;
        sum_slabs_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pa, a, (int64_t)oi, splits, T(1) / T(N));
        return cudaGetLastError();
    }
    EdgePlan p = plan_edge<T, false>(N, I, O, R);
    if (!ws || ws_bytes < (size_t)p.splits * oi * sizeof(T)) return cudaErrorMemoryAllocation;
    T* pa = reinterpret_cast<T*>(ws);
    cudaError_t e = cudaSuccess;
    KAN_EDGE_K(k, (e = launch_edge_param<T, false, KK>(p, s, nullptr, bw, W, nullptr, pa, nullptr, nullptr, N, I, O, R,
                                                       st, x, grid)));
    if (e != cudaSuccess) return e;
    sum_slabs_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pa, a, (int64_t)oi, p.splits, T(1) / T(N));
    return cudaGetLastError();
}

// gx: input gradient through the basis (and through silu when s is NULL); ds: gradient of the
// caller's base values (only with s); dbw, dW: parameter gradients.  NULL = not needed.
template <typename T>
cudaError_t edge_abs_mean_x_bwd(const T* ga, const T* x, const T* s, const T* grid, const T* bw, const T* W,
                                T* gx, T* ds, T* dbw, T* dW, int64_t N, int I, int O, int R, int k,
                                void* ws, size_t ws_bytes, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    const size_t oi = (size_t)O * I;
    if (narrow_applies(N, O, R)) {
        // one kernel for all gradients of a layer with a handful of outputs
        const bool want_param = (dbw && bw) || dW;
        const int splits = narrow_splits(N, I);
        if (want_param && (!ws || ws_bytes < (size_t)splits * oi * (R + 1) * sizeof(T))) return cudaErrorMemoryAllocation;
        T* pdW = reinterpret_cast<T*>(ws);
        T* pdbw = want_param ? pdW + (size_t)splits * oi * R : nullptr;
        e = launch_edge_narrow<T, true>(x, s, grid, bw, W, ga, nullptr, dW ? pdW : nullptr, (dbw && bw) ? pdbw : nullptr,
                                        gx, (ds && s && bw) ? ds : nullptr, N, I, O, R, k, splits, st);
        if (e != cudaSuccess) return e;
        if (dW) {
            sum_slabs_kernel<T><<<grid_1d((int64_t)oi * R, 256), 256, 0, st>>>(pdW, dW, (int64_t)oi * R, splits, T(1));
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        if (dbw && bw) {
            sum_slabs_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pdbw, dbw, (int64_t)oi, splits, T(1));
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    if ((dbw && bw) || dW) {
        EdgePlan p = plan_edge<T, true>(N, I, O, R);
        if (!ws || ws_bytes < (size_t)p.splits * oi * (R + 1) * sizeof(T)) return cudaErrorMemoryAllocation;
        T* pdW = reinterpret_cast<T*>(ws);
        T* pdbw = pdW + (size_t)p.splits * oi * R;
        KAN_EDGE_K(k, (e = launch_edge_param<T, true, KK>(p, s, nullptr, bw, W, ga, nullptr,
                                                          (dbw && bw) ? pdbw : nullptr, dW ? pdW : nullptr, N, I, O,
                                                          R, st, x, grid)));
        if (e != cudaSuccess) return e;
        if (dW) {
            sum_slabs_kernel<T><<<grid_1d((int64_t)oi * R, 256), 256, 0, st>>>(pdW, dW, (int64_t)oi * R, p.splits, T(1));
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        if (dbw && bw) {
            sum_slabs_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pdbw, dbw, (int64_t)oi, p.splits, T(1));
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
    }
    if (gx || (ds && s && bw)) {
        KAN_EDGE_K(k, (e = launch_edge_input<T, KK>(s, nullptr, bw, W, ga, (ds && s && bw) ? ds : nullptr, nullptr, N, I,
                                                    O, R, st, x, grid, gx)));
    }
    return e;
}

// ---------------------------------------------------------------------------
// Edge statistic without caller-provided scratch
// ---------------------------------------------------------------------------
// Fixed scratch for kanb200_edge_abs_mean_noalloc: the per-split partial sums of the forward
// statistic.  4 MiB per GPU that loads the library, held until the process exits.
constexpr size_t kStaticEdgeScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_edge_scratch[kStaticEdgeScratchBytes];

size_t edge_static_scratch_bytes() { return kStaticEdgeScratchBytes; }

// Device address of g_edge_scratch on the CURRENT device.  In host code the symbol is only a
// handle, so the address is looked up once per device (cudaGetSymbolAddress) and cached.
cudaError_t edge_static_scratch(void** ptr) {
    constexpr int kMaxDevices = 64;
    static void* cached[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    void* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        e = cudaGetSymbolAddress(&p, g_edge_scratch);
        if (e != cudaSuccess) return e;
        __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);      // same value from every thread
    }
    *ptr = p;
    return cudaSuccess;
}

// ---------------------------------------------------------------------------
// Scalar head of the activation regulariser (reference: regularization_from_edge_means,
// spline_kan/reference_backend.py:149-170):
//   value = mu1 A + mu2 S,   A = sum a,   p = max(a / max(A, tiny), tiny),   S = -sum p log p
// and its gradient in closed form,  d value / d a_j = mu1 - mu2 (log p_j + S) / A  (entries clamped at
// `tiny` only feel the entropy through A: mu1 + mu2 (1 - S) / A; with A itself clamped nothing but mu1
// is left).  One block, three passes over a (the statistic has O x I entries: at most a few million),
// sums in float64: one launch instead of the twenty-odd elementwise / reduction launches of the
// tensor formulation.
// ---------------------------------------------------------------------------
constexpr int PEN_THREADS = 1024;

__device__ __forceinline__ double block_sum(double v, double* red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                       // red may still be read from the previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < PEN_THREADS / 32; ++w) t += red[w];    // same order in every thread
    return t;
}

template <typename T>
__global__ void __launch_bounds__(PEN_THREADS)
edge_penalty_kernel(const T* __restrict__ a, int64_t n, double mu1, double mu2, T tiny, T* __restrict__ value,
                    T* __restrict__ grad) {
    __shared__ double red[PEN_THREADS / 32];
    double part = 0.0;
    for (int64_t j = threadIdx.x; j < n; j += PEN_THREADS) part += (double)a[j];
    const T total = (T)block_sum(part, red);
    const T safe = total > tiny ? total : tiny;
    part = 0.0;
    for (int64_t j = threadIdx.x; j < n; j += PEN_THREADS) {
        const T q = a[j] / safe;
        const T pj = q > tiny ? q : tiny;
        part += (double)(pj * log(pj));
    }
    const T entropy = (T)(-block_sum(part, red));
    if (threadIdx.x == 0) *value = (T)(mu1 * (double)total + mu2 * (double)entropy);
    if (!grad) return;
    const T m1 = (T)mu1, m2 = (T)mu2;
    const T dead = m1 + (total >= tiny ? m2 * ((T)1 - entropy) / safe : (T)0);
    for (int64_t j = threadIdx.x; j < n; j += PEN_THREADS) {
        const T q = a[j] / safe;
        grad[j] = q >= tiny ? m1 - m2 * (log(q) + entropy) / safe : dead;
    }
}

// The same in two launches that use the whole GPU (a statistic of 200 000 entries keeps the single block
// above busy for 60 us).  With q = a / A,  sum q log q = (sum a log a - log A sum a) / A, so ONE pass
// gives A and the entropy: every block leaves (sum a, sum a log a, number of zero entries) in the
// workspace; the second kernel's blocks each add those partial sums in the same fixed order, block 0
// writes the value and all of them write their share of the gradient, with the clamps decided per
// element as above.  (An entry below tiny * A but above zero -- a denormal next to normal entries --
// enters the entropy with its own q log q instead of tiny log tiny: a difference of 1e-36.)
constexpr int PEN2_THREADS = 256, PEN2_MAX_BLOCKS = 256;
constexpr size_t kPenaltyWorkspaceBytes = (size_t)PEN2_MAX_BLOCKS * 3 * sizeof(double);

template <int THREADS>
__device__ __forceinline__ void block_sum3(double (&v)[3], double (*red)[3]) {
#pragma unroll
    for (int c = 0; c < 3; ++c)
        for (int o = 16; o > 0; o >>= 1) v[c] += __shfl_xor_sync(0xffffffffu, v[c], o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
        for (int c = 0; c < 3; ++c) red[warp][c] = v[c];
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        double t = 0.0;
        for (int w = 0; w < THREADS / 32; ++w) t += red[w][c];
        v[c] = t;
    }
}

template <typename T>
__global__ void __launch_bounds__(PEN2_THREADS)
edge_penalty_partial_kernel(const T* __restrict__ a, int64_t n, double* __restrict__ partial) {
    __shared__ double red[PEN2_THREADS / 32][3];
    double v[3] = {0.0, 0.0, 0.0};
    for (int64_t j = (int64_t)blockIdx.x * PEN2_THREADS + threadIdx.x; j < n; j += (int64_t)gridDim.x * PEN2_THREADS) {
        const T aj = a[j];
        if (aj > T(0)) {
            v[0] += (double)aj;
            v[1] += (double)(aj * log(aj));
        } else {
            v[2] += 1.0;
        }
    }
    block_sum3<PEN2_THREADS>(v, red);
    if (threadIdx.x == 0)
        for (int c = 0; c < 3; ++c) partial[(size_t)blockIdx.x * 3 + c] = v[c];
}

template <typename T>
__global__ void __launch_bounds__(PEN2_THREADS)
edge_penalty_finish_kernel(const T* __restrict__ a, int64_t n, const double* __restrict__ partial, int n_partial,
                           double mu1, double mu2, T tiny, T* __restrict__ value, T* __restrict__ grad) {
    __shared__ double red[PEN2_THREADS / 32][3];
    double v[3] = {0.0, 0.0, 0.0};
    for (int b = threadIdx.x; b < n_partial; b += PEN2_THREADS)          // same order in every block
        for (int c = 0; c < 3; ++c) v[c] += partial[(size_t)b * 3 + c];
    block_sum3<PEN2_THREADS>(v, red);
    const T total = (T)v[0];
    const T safe = total > tiny ? total : tiny;
    // -sum p log p: entries above zero with their own q log q, zero entries clamped at tiny
    const double ent = -((v[1] - log((double)safe) * v[0]) / (double)safe) - v[2] * ((double)tiny * log((double)tiny));
    const T entropy = (T)ent;
    if (blockIdx.x == 0 && threadIdx.x == 0) *value = (T)(mu1 * (double)total + mu2 * (double)entropy);
    if (!grad) return;
    const T m1 = (T)mu1, m2 = (T)mu2;
    const T dead = m1 + (total >= tiny ? m2 * ((T)1 - entropy) / safe : (T)0);
    for (int64_t j = (int64_t)blockIdx.x * PEN2_THREADS + threadIdx.x; j < n; j += (int64_t)gridDim.x * PEN2_THREADS) {
        const T q = a[j] / safe;
        grad[j] = q >= tiny ? m1 - m2 * (log(q) + entropy) / safe : dead;
    }
}

size_t edge_penalty_workspace_bytes() { return kPenaltyWorkspaceBytes; }

template <typename T>
cudaError_t edge_penalty(const T* a, int64_t n, double mu1, double mu2, T* value, T* grad, void* ws, size_t ws_bytes,
                         cudaStream_t st) {
    const T tiny = sizeof(T) == 4 ? (T)1.17549435e-38 : (T)2.2250738585072014e-308;
    if (!ws || ws_bytes < kPenaltyWorkspaceBytes || n < 4096) {
        edge_penalty_kernel<T><<<1, PEN_THREADS, 0, st>>>(a, n, mu1, mu2, tiny, value, grad);
        return cudaGetLastError();
    }
    int64_t blocks = (n + 4 * PEN2_THREADS - 1) / (4 * PEN2_THREADS);
    if (blocks > PEN2_MAX_BLOCKS) blocks = PEN2_MAX_BLOCKS;
    double* partial = reinterpret_cast<double*>(ws);
    edge_penalty_partial_kernel<T><<<(int)blocks, PEN2_THREADS, 0, st>>>(a, n, partial);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    edge_penalty_finish_kernel<T><<<(int)blocks, PEN2_THREADS, 0, st>>>(a, n, partial, (int)blocks, mu1, mu2, tiny, value,
                                                                          grad);
    return cudaGetLastError();
}
template cudaError_t edge_penalty<float>(const float*, int64_t, double, double, float*, float*, void*, size_t,
                                         cudaStream_t);
template cudaError_t edge_penalty<double>(const double*, int64_t, double, double, double*, double*, void*, size_t,
                                          cudaStream_t);

// ---------------------------------------------------------------------------
// Layer forward / backward for at most 16 outputs (any float type, k <= 3, R <= 16)
// ---------------------------------------------------------------------------
bool narrow_layer_supported(int O, int R, int k) { return O >= 1 && O <= kNarrowMaxO && R <= 16 && k >= 1 && k <= 3; }

template <typename T>
size_t narrow_layer_workspace(int64_t N, int I, int O, int R) {
    return (size_t)narrow_splits(N, I) * (size_t)O * I * (size_t)(R + 1) * sizeof(T);
}

template <typename T>
cudaError_t narrow_layer_forward(const T* x, const T* grid, const T* bw, const T* sw, const T* scaler, T* y, int64_t N,
                                 int I, int O, int R, int k, cudaStream_t st) {
    if (N < 1) return cudaSuccess;
    const int blocks = (int)((N + NF_ROWS - 1) / NF_ROWS);
    constexpr int OT = sizeof(T) == 4 ? 16 : 8;
    if (O <= 4) {
        KAN_EDGE_K(k, (narrow_layer_forward_kernel<T, KK, 4><<<blocks, EN_THREADS, 0, st>>>(x, grid, bw, sw, scaler, y, N,
                                                                                           I, O, R)));
    } else {
        KAN_EDGE_K(k, (narrow_layer_forward_kernel<T, KK, OT><<<blocks, EN_THREADS, 0, st>>>(x, grid, bw, sw, scaler, y,
                                                                                            N, I, O, R)));
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t narrow_layer_backward(const T* dY, const T* x, const T* grid, const T* bw, const T* sw, const T* scaler,
                                  T* gx, T* gbw, T* gsw, T* gscaler, int64_t N, int I, int O, int R, int k, void* ws,
                                  size_t ws_bytes, cudaStream_t st) {
    if (N < 1) return cudaSuccess;
    const bool want_param = gsw || gscaler || (gbw && bw);
    const int splits = narrow_splits(N, I);
    const size_t oi = (size_t)O * I;
    if (want_param && (!ws || ws_bytes < narrow_layer_workspace<T>(N, I, O, R))) return cudaErrorMemoryAllocation;
    T* pdW = reinterpret_cast<T*>(ws);
    T* pdbw = want_param ? pdW + (size_t)splits * oi * R : nullptr;
    const int64_t rows = (N + splits - 1) / splits;
    const dim3 blocks(I, splits);
    T* pw = (gsw || gscaler) ? pdW : nullptr;
    T* pb = (gbw && bw) ? pdbw : nullptr;
    // accumulators per thread: outputs x (slots + 1); float 8 x 9 or 4 x 17, double 4 x 9 or 2 x 17
    if (R <= EN_R) {
        constexpr int OT = sizeof(T) == 4 ? 8 : 4;
        KAN_EDGE_K(k, (edge_narrow_kernel<T, KK, OT, true, EN_R, true><<<blocks, EN_THREADS, 0, st>>>(
                          x, nullptr, grid, bw, sw, dY, nullptr, pw, pb, gx, nullptr, N, I, O, R, rows, scaler)));
    } else {
        constexpr int OT = sizeof(T) == 4 ? 4 : 2;
        KAN_EDGE_K(k, (edge_narrow_kernel<T, KK, OT, true, 16, true><<<blocks, EN_THREADS, 0, st>>>(
                          x, nullptr, grid, bw, sw, dY, nullptr, pw, pb, gx, nullptr, N, I, O, R, rows, scaler)));
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || !want_param) return e;
    narrow_layer_finalize_kernel<T><<<grid_1d((int64_t)oi, 256), 256, 0, st>>>(pdW, pdbw, sw, scaler, gsw, gscaler,
                                                                              (gbw && bw) ? gbw : nullptr, (int64_t)oi, R,
                                                                              splits);
    return cudaGetLastError();
}

#define KAN_INSTANTIATE(T)                                                                               \
    template size_t edge_workspace<T>(int64_t, int, int, int, bool);                                     \
    template cudaError_t edge_abs_mean_fwd<T>(const T*, const T*, const T*, const T*, T*, int64_t, int,  \
                                              int, int, void*, size_t, cudaStream_t);                    \
    template cudaError_t edge_abs_mean_bwd<T>(const T*, const T*, const T*, const T*, const T*, T*, T*,  \
                                              T*, T*, int64_t, int, int, int, void*, size_t, cudaStream_t); \
    template cudaError_t edge_abs_mean_x_fwd<T>(const T*, const T*, const T*, const T*, const T*, T*, int64_t, \
                                                int, int, int, int, void*, size_t, cudaStream_t);         \
    template cudaError_t edge_abs_mean_x_bwd<T>(const T*, const T*, const T*, const T*, const T*, const T*, T*, \
                                                T*, T*, T*, int64_t, int, int, int, int, void*, size_t, cudaStream_t);
KAN_INSTANTIATE(float)
KAN_INSTANTIATE(double)
#define KAN_INSTANTIATE_NARROW(T)                                                                              \
    template size_t narrow_layer_workspace<T>(int64_t, int, int, int);                                         \
    template cudaError_t narrow_layer_forward<T>(const T*, const T*, const T*, const T*, const T*, T*, int64_t, int,  \
                                                 int, int, int, cudaStream_t);                                 \
    template cudaError_t narrow_layer_backward<T>(const T*, const T*, const T*, const T*, const T*, const T*, T*, T*, \
                                                  T*, T*, int64_t, int, int, int, int, void*, size_t, cudaStream_t);
KAN_INSTANTIATE_NARROW(float)
KAN_INSTANTIATE_NARROW(double)

}  // namespace kanb200
