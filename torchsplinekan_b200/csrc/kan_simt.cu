// SIMT (FMA-pipe) kernels of the KANLinear path, templated on float / double.
//
// They serve float64 (no tensor-core kind exists for it), shapes the
// tensor-core path does not take (tiny layers, wide grids) and the standalone
// basis / basis-gradient operators.  All of them evaluate only the k+1
// non-zero basis functions of each input ("gather" formulation) and none uses
// global atomics: reductions over samples go through per-split partial slabs
// in the caller's workspace and a fixed-order second pass.
#include "kan_device.cuh"
#include "kan_internal.h"
#include "kan_table.cuh"

namespace kanb200 {

namespace {

// ---------------------------------------------------------------------------
// Dense basis  H[n,i,:]   (HBM-bound: 4 N I (R+1) bytes for float)
// ---------------------------------------------------------------------------
// A block evaluates P consecutive (n,i) pairs, assembles their dense rows in
// shared memory and streams them out with fully coalesced stores.
template <typename T, int K>
__global__ void basis_kernel(const T* __restrict__ x, const T* __restrict__ grid, T* __restrict__ H,
                             int64_t pairs, int I, int G) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* rows = reinterpret_cast<T*>(smem_raw);
    const int R = G + K, nk = G + 2 * K + 1;
    const int P = blockDim.x;
    for (int64_t base = (int64_t)blockIdx.x * P; base < pairs; base += (int64_t)gridDim.x * P) {
        const int64_t idx = base + threadIdx.x;
        T* row = rows + (size_t)threadIdx.x * R;
        for (int r = 0; r < R; ++r) row[r] = T(0);
        if (idx < pairs) {
            const int i = (int)(idx % I);
            const T* t = grid + (size_t)i * nk;
            const T xv = x[idx];
            const int m = locate_span(t, nk, xv);
            if (m >= 0) {
                T v[K + 1], d[K + 1];
                window_values<K, T, false>(t, nk, m, xv, v, d);
#pragma unroll
                for (int j = 0; j <= K; ++j) {
                    const int r = m - K + j;
                    if (r >= 0 && r < R) row[r] = v[j];
                }
            }
        }
        __syncthreads();
        const int64_t left = pairs - base;
        const int64_t cnt = (left < P ? left : P) * R;
        T* out = H + base * R;
        for (int64_t e = threadIdx.x; e < cnt; e += P) out[e] = rows[e];
        __syncthreads();
    }
}

// R == 8, float: one pair per lane, then the warp's 32 rows (1 KB) leave as 64 float4 in two fully
// coalesced store instructions; the row pieces are fetched from the owning lane by shuffles.
template <int K>
__global__ void __launch_bounds__(256)
basis_r8_kernel(const float* __restrict__ x, const float* __restrict__ grid, float* __restrict__ H,
                int64_t pairs, int I, int G) {
    const int nk = G + 2 * K + 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t wbase = ((int64_t)blockIdx.x * (blockDim.x >> 5) + warp) * 32; wbase < pairs;
         wbase += warps_total * 32) {
        const int64_t idx = wbase + lane;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        int s = 0;
        if (idx < pairs) {
            const int i = (int)(idx % I);
            const float* t = grid + (size_t)i * nk;           // knot rows stay in L1
            const float xv = x[idx];
            const int m = locate_span(t, nk, xv);
            if (m >= 0) {
                float w[K + 1], d[K + 1];
                window_values<K, float, false>(t, nk, m, xv, w, d);
                s = m - K;
#pragma unroll
                for (int j = 0; j <= K; ++j) v[j] = w[j];
            } else {
                s = -100;                                  // nothing lands in [0, 8)
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int q4 = lane + 32 * h;                  // float4 index within the warp's 64
            const int src = q4 >> 1;                       // lane that owns the pair
            const int r0 = (q4 & 1) * 4;                   // first slot of this float4
            float pv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) pv[j] = __shfl_sync(0xffffffffu, v[j], src);
            const int ps = __shfl_sync(0xffffffffu, s, src);
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = r0 + e - ps;                 // index into the window, valid 0..K
                float val = 0.f;
#pragma unroll
                for (int jj = 0; jj <= K; ++jj) val = (j == jj) ? pv[jj] : val;
                o[e] = val;
            }
            if (wbase + src < pairs)
                reinterpret_cast<float4*>(H + wbase * 8)[q4] = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

// R == 8, float: each lane reads its whole 32-byte gradient row with two 16-byte loads.
template <int K>
__global__ void __launch_bounds__(256)
basis_grad_r8_kernel(const float* __restrict__ x, const float* __restrict__ grid, const float* __restrict__ gH,
                     float* __restrict__ gx, int64_t pairs, int I, int G) {
    const int nk = G + 2 * K + 1;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < pairs;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % I);
        const float* t = grid + (size_t)i * nk;
        const float4 a = __ldg(reinterpret_cast<const float4*>(gH + idx * 8));
        const float4 b = __ldg(reinterpret_cast<const float4*>(gH + idx * 8) + 1);
        const float g[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        const float xv = x[idx];
        const int m = locate_span(t, nk, xv);
        float acc = 0.f;
        if (m >= 0) {
            float v[K + 1], d[K + 1];
            window_values<K, float, true>(t, nk, m, xv, v, d);
#pragma unroll
            for (int j = 0; j <= K; ++j) {
                const int r = m - K + j;
                float gr = 0.f;
#pragma unroll
                for (int q = 0; q < 8; ++q) gr = (r == q) ? g[q] : gr;
                acc += gr * d[j];
            }
        }
        gx[idx] = acc;
    }
}

// ---------------------------------------------------------------------------
// Table-driven basis kernels (float, R == 8, at most 12 knots).
//
// A block owns 32 consecutive features and a range of rows; lane = feature.  The lane keeps its
// feature's knots in registers and the block keeps the polynomial coefficients of its features'
// spans (kan_table.cuh, built once per call by the table kernel into the caller's workspace) in
// shared memory.  Per value: one coalesced read of x, a compare-and-count span search in
// registers, four 16-byte shared-memory loads and a Horner evaluation.  The warp's 32 basis rows
// (1 KB, contiguous in H) leave as 64 float4 in two coalesced stores.
// Shared-memory layout: feature stride 356 floats (= 4 mod 32), span stride 32 floats, so the
// 16-byte loads of a quarter-warp hit distinct banks whatever spans its lanes are in.
// ---------------------------------------------------------------------------
constexpr int BT_FEATURES = 32, BT_SPANS = 11, BT_SPAN_STRIDE = 32, BT_STRIDE = BT_SPANS * BT_SPAN_STRIDE + 4;
constexpr int BT_THREADS = 256, BT_UNROLL = 4;

// Copies the coefficients of the block's 32 features from the table (per feature `fs` floats:
// 16 of header and knots, then 20 per span of which the first 16 are coefficients).
__device__ __forceinline__ void basis_table_fill(float* __restrict__ stab, const float* __restrict__ tab,
                                                 int fs, int nk, int f0, int I) {
    const int spans = nk - 1;
    for (int idx = threadIdx.x; idx < BT_FEATURES * spans * 4; idx += blockDim.x) {
        const int q = idx & 3;                  // which 16-byte piece (coefficients of function q)
        const int e = (idx >> 2) % spans, fl = (idx >> 2) / spans;
        const int f = (f0 + fl < I) ? f0 + fl : I - 1;
        const float4 v = __ldg(reinterpret_cast<const float4*>(tab + (size_t)f * fs + 16 + e * TAB_ENTRY_FLOATS) + q);
        *reinterpret_cast<float4*>(stab + fl * BT_STRIDE + e * BT_SPAN_STRIDE + q * 4) = v;
    }
    __syncthreads();
}

// The lane's knots: t_0 .. t_{nk-2} padded with +inf (kn[0..10]) and the last knot.
struct LaneKnots {
    float kn[11];
    float last;
};

__device__ __forceinline__ LaneKnots load_lane_knots(const float* __restrict__ ftab_global) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(ftab_global + 4));
    const float4 b = __ldg(reinterpret_cast<const float4*>(ftab_global + 4) + 1);
    const float4 c = __ldg(reinterpret_cast<const float4*>(ftab_global + 4) + 2);
    LaneKnots k;
    k.kn[0] = a.x; k.kn[1] = a.y; k.kn[2] = a.z; k.kn[3] = a.w;
    k.kn[4] = b.x; k.kn[5] = b.y; k.kn[6] = b.z; k.kn[7] = b.w;
    k.kn[8] = c.x; k.kn[9] = c.y; k.kn[10] = c.z;
    k.last = c.w;
    return k;
}

// DERIV = false: the k+1 window values; true: their derivatives.  Returns the window start
// (K = spline order); inputs outside the knot range (or NaN) give zeros.
template <bool DERIV>
__device__ __forceinline__ int basis_table_eval(const float* __restrict__ fcoef, const LaneKnots& k, int K,
                                                float xv, float (&v)[4]) {
    const bool inside = (xv >= k.kn[0]) && (xv <= k.last);
    int m = 0;
    float tm = k.kn[0];
#pragma unroll
    for (int q = 1; q < 11; ++q) {
        const bool ge = xv >= k.kn[q];
        m += ge ? 1 : 0;
        tm = ge ? k.kn[q] : tm;                 // knots are non-decreasing: ends at t_m
    }
    m = inside ? m : 0;
    const float4* ent = reinterpret_cast<const float4*>(fcoef + m * BT_SPAN_STRIDE);
    const float4 c0 = ent[0], c1 = ent[1], c2 = ent[2], c3 = ent[3];
    const float u = xv - tm;
    if (DERIV) {
        v[0] = fmaf(fmaf(3.0f * c0.w, u, 2.0f * c0.z), u, c0.y);
        v[1] = fmaf(fmaf(3.0f * c1.w, u, 2.0f * c1.z), u, c1.y);
        v[2] = fmaf(fmaf(3.0f * c2.w, u, 2.0f * c2.z), u, c2.y);
        v[3] = fmaf(fmaf(3.0f * c3.w, u, 2.0f * c3.z), u, c3.y);
    } else {
        v[0] = fmaf(fmaf(fmaf(c0.w, u, c0.z), u, c0.y), u, c0.x);
        v[1] = fmaf(fmaf(fmaf(c1.w, u, c1.z), u, c1.y), u, c1.x);
        v[2] = fmaf(fmaf(fmaf(c2.w, u, c2.z), u, c2.y), u, c2.x);
        v[3] = fmaf(fmaf(fmaf(c3.w, u, c3.z), u, c3.y), u, c3.x);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = inside ? v[j] : 0.f;
    return m - K;
}

__global__ void __launch_bounds__(BT_THREADS, 4)
basis_table_kernel(const float* __restrict__ x, const float* __restrict__ tab, int fs, float* __restrict__ H,
                   int64_t N, int I, int G, int K, int64_t rows_per_block) {
    __shared__ __align__(16) float stab[BT_FEATURES * BT_STRIDE];
    const int f0 = blockIdx.x * BT_FEATURES;
    const int nk = G + 2 * K + 1;
    basis_table_fill(stab, tab, fs, nk, f0, I);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int f = f0 + lane;
    const float* fcoef = stab + lane * BT_STRIDE;
    const LaneKnots knots = load_lane_knots(tab + (size_t)(f < I ? f : I - 1) * fs);
    const int64_t row0 = (int64_t)blockIdx.y * rows_per_block;
    int64_t row1 = row0 + rows_per_block;
    if (row1 > N) row1 = N;
    const int n_valid = (I - f0 < 32) ? I - f0 : 32;       // features of this group
    // BT_UNROLL rows per warp and iteration: their x loads are issued together
    for (int64_t rbase = row0 + warp * BT_UNROLL; rbase < row1; rbase += (BT_THREADS / 32) * BT_UNROLL) {
        float xv[BT_UNROLL];
#pragma unroll
        for (int u = 0; u < BT_UNROLL; ++u)
            xv[u] = (f < I && rbase + u < row1) ? __ldg(x + (size_t)(rbase + u) * I + f) : 0.f;
#pragma unroll
        for (int u = 0; u < BT_UNROLL; ++u) {
            const int64_t row = rbase + u;
            if (row >= row1) break;                         // uniform over the warp
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            int s = -100;                                   // nothing lands in [0, 8)
            if (f < I) s = basis_table_eval<false>(fcoef, knots, K, xv[u], v);
            float4* dst = reinterpret_cast<float4*>(H + ((size_t)row * I + f0) * 8);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int q4 = lane + 32 * h;               // float4 index within the warp's 64
                const int src = q4 >> 1;                    // lane that owns the pair
                const int r0 = (q4 & 1) * 4;                // first slot of this float4
                float pv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) pv[j] = __shfl_sync(0xffffffffu, v[j], src);
                const int ps = __shfl_sync(0xffffffffu, s, src);
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = r0 + e - ps;              // index into the window
                    float val = 0.f;
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) val = (j == jj) ? pv[jj] : val;
                    o[e] = val;
                }
                if (src < n_valid) dst[q4] = make_float4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

__global__ void __launch_bounds__(BT_THREADS, 4)
basis_grad_table_kernel(const float* __restrict__ x, const float* __restrict__ tab, int fs,
                        const float* __restrict__ gH, float* __restrict__ gx, int64_t N, int I, int G, int K,
                        int64_t rows_per_block) {
    __shared__ __align__(16) float stab[BT_FEATURES * BT_STRIDE];
    const int f0 = blockIdx.x * BT_FEATURES;
    const int nk = G + 2 * K + 1;
    basis_table_fill(stab, tab, fs, nk, f0, I);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int f = f0 + lane;
    const float* fcoef = stab + lane * BT_STRIDE;
    const LaneKnots knots = load_lane_knots(tab + (size_t)(f < I ? f : I - 1) * fs);
    const int64_t row0 = (int64_t)blockIdx.y * rows_per_block;
    int64_t row1 = row0 + rows_per_block;
    if (row1 > N) row1 = N;
    if (f >= I) return;                                     // no warp-wide operation below
    for (int64_t rbase = row0 + warp * BT_UNROLL; rbase < row1; rbase += (BT_THREADS / 32) * BT_UNROLL) {
        float xv[BT_UNROLL];
        float4 ga[BT_UNROLL], gb[BT_UNROLL];
#pragma unroll
        for (int u = 0; u < BT_UNROLL; ++u) {
            const bool ok = rbase + u < row1;
            const size_t idx = (size_t)(ok ? rbase + u : row0) * I + f;
            xv[u] = __ldg(x + idx);
            ga[u] = __ldg(reinterpret_cast<const float4*>(gH + idx * 8));
            gb[u] = __ldg(reinterpret_cast<const float4*>(gH + idx * 8) + 1);
        }
#pragma unroll
        for (int u = 0; u < BT_UNROLL; ++u) {
            if (rbase + u >= row1) break;
            const float g[8] = {ga[u].x, ga[u].y, ga[u].z, ga[u].w, gb[u].x, gb[u].y, gb[u].z, gb[u].w};
            float d[4];
            const int s = basis_table_eval<true>(fcoef, knots, K, xv[u], d);
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = s + j;
                float gr = 0.f;
#pragma unroll
                for (int q = 0; q < 8; ++q) gr = (r == q) ? g[q] : gr;
                acc = fmaf(gr, d[j], acc);
            }
            gx[(size_t)(rbase + u) * I + f] = acc;
        }
    }
}

template <typename T, int K>
__global__ void basis_grad_kernel(const T* __restrict__ x, const T* __restrict__ grid,
                                  const T* __restrict__ gH, T* __restrict__ gx,
                                  int64_t pairs, int I, int G) {
    const int R = G + K, nk = G + 2 * K + 1;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < pairs;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % I);
        const T* t = grid + (size_t)i * nk;
        const T xv = x[idx];
        const int m = locate_span(t, nk, xv);
        T acc = T(0);
        if (m >= 0) {
            T v[K + 1], d[K + 1];
            window_values<K, T, true>(t, nk, m, xv, v, d);
            const T* g = gH + idx * R;
#pragma unroll
            for (int j = 0; j <= K; ++j) {
                const int r = m - K + j;
                if (r >= 0 && r < R) acc += g[r] * d[j];
            }
        }
        gx[idx] = acc;
    }
}

// ---------------------------------------------------------------------------
// Forward:  y[n,o] = sum_i ( silu(x) bw[o,i] + sum_j val_j W_eff[o,i,s+j] )
// ---------------------------------------------------------------------------
constexpr int FW_TN = 32, FW_TO = 64, FW_NPT = 8, FW_THREADS = 256;

template <typename T>
struct FwdSmem {
    int CI, RW, K1, nk;
    __host__ __device__ size_t w_elems() const { return (size_t)CI * RW * (FW_TO + 1); }
    __host__ __device__ size_t vals_elems() const { return (size_t)FW_TN * CI * K1; }
    __host__ __device__ size_t sil_elems() const { return (size_t)FW_TN * CI; }
    __host__ __device__ size_t knot_elems() const { return (size_t)CI * nk; }
    __host__ __device__ size_t bytes() const {
        return (w_elems() + vals_elems() + sil_elems() + knot_elems()) * sizeof(T) +
               (size_t)FW_TN * CI * sizeof(int) + 16;
    }
};

template <typename T, int K>
__global__ void __launch_bounds__(FW_THREADS)
fwd_simt_kernel(const T* __restrict__ x, const T* __restrict__ grid, const T* __restrict__ bw,
                const T* __restrict__ sw, const T* __restrict__ scaler, T* __restrict__ y,
                int64_t N, int I, int O, int G, int CI) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = G + K, nk = G + 2 * K + 1, RW = R + 1;
    FwdSmem<T> L{CI, RW, K + 1, nk};
    T* Wt = reinterpret_cast<T*>(smem_raw);                  // [CI][RW][TO+1]
    T* vals = Wt + L.w_elems();                              // [TN][CI][K+1]
    T* sil = vals + L.vals_elems();                          // [TN][CI]
    T* knots = sil + L.sil_elems();                          // [CI][nk]
    int* st = reinterpret_cast<int*>(knots + L.knot_elems()); // [TN][CI]

    const int tid = threadIdx.x;
    const int to = tid & (FW_TO - 1);
    const int ng = tid / FW_TO;
    const int o0 = blockIdx.y * FW_TO;
    const int64_t n0 = (int64_t)blockIdx.x * FW_TN;

    T acc[FW_NPT];
#pragma unroll
    for (int q = 0; q < FW_NPT; ++q) acc[q] = T(0);

    for (int i0 = 0; i0 < I; i0 += CI) {
        const int ci = (I - i0 < CI) ? (I - i0) : CI;
        __syncthreads();
        for (int e = tid; e < ci * nk; e += FW_THREADS) knots[e] = grid[(size_t)i0 * nk + e];
        for (int e = tid; e < FW_TO * ci * R; e += FW_THREADS) {
            const int o = e / (ci * R);
            const int rem = e - o * (ci * R);
            const int i = rem / R, r = rem - i * R;
            T w = T(0);
            if (o0 + o < O) {
                const size_t oi = (size_t)(o0 + o) * I + (i0 + i);
                w = sw[oi * R + r];
                if (scaler) w *= scaler[oi];
            }
            Wt[((size_t)i * RW + r) * (FW_TO + 1) + o] = w;
        }
        for (int e = tid; e < FW_TO * ci; e += FW_THREADS) {
            const int o = e / ci, i = e - o * ci;
            T w = T(0);
            if (bw && o0 + o < O) w = bw[(size_t)(o0 + o) * I + (i0 + i)];
            Wt[((size_t)i * RW + R) * (FW_TO + 1) + o] = w;
        }
        __syncthreads();
        for (int e = tid; e < FW_TN * ci; e += FW_THREADS) {
            const int n = e / ci, i = e - n * ci;
            T w[K + 1];
            int s = 0;
            T sv = T(0);
#pragma unroll
            for (int j = 0; j <= K; ++j) w[j] = T(0);
            if (n0 + n < N) {
                const T xv = x[(size_t)(n0 + n) * I + (i0 + i)];
                const T* t = knots + (size_t)i * nk;
                const int m = locate_span(t, nk, xv);
                if (m >= 0) {
                    T v[K + 1], d[K + 1];
                    window_values<K, T, false>(t, nk, m, xv, v, d);
                    s = window_in_range<K, T>(m, R, v, w);
                }
                sv = bw ? silu_t<T>(xv) : T(0);
            }
#pragma unroll
            for (int j = 0; j <= K; ++j) vals[((size_t)n * CI + i) * (K + 1) + j] = w[j];
            sil[(size_t)n * CI + i] = sv;
            st[(size_t)n * CI + i] = s;
        }
        __syncthreads();
        for (int i = 0; i < ci; ++i) {
            const T* wcol = Wt + (size_t)i * RW * (FW_TO + 1) + to;
            const T wb = wcol[(size_t)R * (FW_TO + 1)];
#pragma unroll
            for (int q = 0; q < FW_NPT; ++q) {
                const int n = ng * FW_NPT + q;
                const int s = st[(size_t)n * CI + i];
                const T* vp = vals + ((size_t)n * CI + i) * (K + 1);
                const T* wp = wcol + (size_t)s * (FW_TO + 1);
                T a = acc[q];
#pragma unroll
                for (int j = 0; j <= K; ++j) a += vp[j] * wp[(size_t)j * (FW_TO + 1)];
                a += sil[(size_t)n * CI + i] * wb;
                acc[q] = a;
            }
        }
    }
    if (o0 + to < O) {
#pragma unroll
        for (int q = 0; q < FW_NPT; ++q) {
            const int64_t n = n0 + ng * FW_NPT + q;
            if (n < N) y[(size_t)n * O + o0 + to] = acc[q];
        }
    }
}

// ---------------------------------------------------------------------------
// Backward, parameters:  D[o,i,r] = sum_n dY[n,o] H[n,i,r],  Db[o,i] = sum_n dY[n,o] silu(x[n,i])
// ---------------------------------------------------------------------------
// Thread owns OPT outputs x one feature with the whole R+1 row of accumulators
// in registers; dense rows of H for a tile of samples are rebuilt in shared
// memory from x.  One slab of partial sums per sample split.
constexpr int BP_TI = 4, BP_THREADS = 128;

template <typename T, int K, int RMAX, int OPT, int TNS>
__global__ void __launch_bounds__(BP_THREADS)
bwd_param_simt_kernel(const T* __restrict__ dY, const T* __restrict__ x, const T* __restrict__ grid,
                      T* __restrict__ partial, int64_t N, int I, int O, int G, bool has_base,
                      int64_t n_per_split) {
    constexpr int RS = RMAX + 1;                 // row: RMAX spline slots + base slot
    constexpr int TO = 32 * OPT;
    __shared__ T Hs[TNS][BP_TI][RS];
    __shared__ T dYs[TNS][TO];
    __shared__ T knots[BP_TI][kMaxKnots];
    const int R = G + K, nk = G + 2 * K + 1;
    const int tid = threadIdx.x;
    const int lane_o = tid & 31, ti = tid >> 5;
    const int o0 = blockIdx.x * TO, i0 = blockIdx.y * BP_TI;
    const int64_t nb = (int64_t)blockIdx.z * n_per_split;
    const int64_t ne = (nb + n_per_split < N) ? nb + n_per_split : N;

    for (int e = tid; e < BP_TI * nk; e += BP_THREADS) {
        const int i = e / nk, q = e - i * nk;
        knots[i][q] = (i0 + i < I) ? grid[(size_t)(i0 + i) * nk + q] : T(0);
    }
    T acc[OPT][RS];
#pragma unroll
    for (int u = 0; u < OPT; ++u)
#pragma unroll
        for (int r = 0; r < RS; ++r) acc[u][r] = T(0);

    for (int64_t nt = nb; nt < ne; nt += TNS) {
        __syncthreads();
        for (int e = tid; e < TNS * TO; e += BP_THREADS) {
            const int n = e / TO, o = e - n * TO;
            dYs[n][o] = (nt + n < ne && o0 + o < O) ? dY[(size_t)(nt + n) * O + o0 + o] : T(0);
        }
        for (int e = tid; e < TNS * BP_TI; e += BP_THREADS) {
            const int n = e / BP_TI, i = e - n * BP_TI;
            T* row = &Hs[n][i][0];
            for (int r = 0; r < RS; ++r) row[r] = T(0);
            if (nt + n < ne && i0 + i < I) {
                const T xv = x[(size_t)(nt + n) * I + i0 + i];
                const int m = locate_span(&knots[i][0], nk, xv);
                if (m >= 0) {
                    T v[K + 1], d[K + 1];
                    window_values<K, T, false>(&knots[i][0], nk, m, xv, v, d);
#pragma unroll
                    for (int j = 0; j <= K; ++j) {
                        const int r = m - K + j;
                        if (r >= 0 && r < R) row[r] = v[j];
                    }
                }
                if (has_base) row[RMAX] = silu_t<T>(xv);
            }
        }
        __syncthreads();
#pragma unroll 2
        for (int n = 0; n < TNS; ++n) {
            T dy[OPT];
#pragma unroll
            for (int u = 0; u < OPT; ++u) dy[u] = dYs[n][lane_o + 32 * u];
            const T* row = &Hs[n][ti][0];
#pragma unroll
            for (int r = 0; r < RS; ++r) {
                const T h = row[r];
#pragma unroll
                for (int u = 0; u < OPT; ++u) acc[u][r] += dy[u] * h;
            }
        }
    }
    if (i0 + ti < I) {
        const int RW = R + 1;
#pragma unroll
        for (int u = 0; u < OPT; ++u) {
            const int o = o0 + lane_o + 32 * u;
            if (o >= O) continue;
            T* out = partial + ((size_t)blockIdx.z * O + o) * ((size_t)I * RW) + (size_t)(i0 + ti) * RW;
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                if (r < R) out[r] = acc[u][r];
            out[R] = acc[u][RMAX];
        }
    }
}

template <typename T>
__global__ void finalize_param_kernel(const T* __restrict__ partial, int splits, int64_t split_stride,
                                      int64_t ldo, int sI, int64_t boff, int sB,
                                      const T* __restrict__ sw, const T* __restrict__ scaler,
                                      T* __restrict__ gsw, T* __restrict__ gscaler, T* __restrict__ gbw,
                                      int O, int I, int R) {
    const int64_t total = (int64_t)O * I;
    for (int64_t oi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; oi < total;
         oi += (int64_t)gridDim.x * blockDim.x) {
        const int o = (int)(oi / I), i = (int)(oi - (int64_t)o * I);
        const T* p0 = partial + (size_t)o * ldo;
        if (gsw || gscaler) {
            const T sc = scaler ? scaler[oi] : T(1);
            T gs = T(0);
            for (int r = 0; r < R; ++r) {
                T d = T(0);
                for (int s = 0; s < splits; ++s) d += p0[(size_t)s * split_stride + (size_t)i * sI + r];
                if (gsw) gsw[(size_t)oi * R + r] = scaler ? sc * d : d;
                if (gscaler) gs += sw[(size_t)oi * R + r] * d;
            }
            if (gscaler) gscaler[oi] = gs;
        }
        if (gbw) {
            T d = T(0);
            for (int s = 0; s < splits; ++s) d += p0[(size_t)s * split_stride + boff + (size_t)i * sB];
            gbw[oi] = d;
        }
    }
}

// The same sums with one warp per (o, i): the lanes stride over the slabs and a butterfly adds
// them up, for plans with many row splits (small layers over long batches).
template <typename T>
__global__ void finalize_param_wide_kernel(const T* __restrict__ partial, int splits, int64_t split_stride,
                                           int64_t ldo, int sI, int64_t boff, int sB,
                                           const T* __restrict__ sw, const T* __restrict__ scaler,
                                           T* __restrict__ gsw, T* __restrict__ gscaler, T* __restrict__ gbw,
                                           int O, int I, int R) {
    const int lane = threadIdx.x & 31;
    const int64_t total = (int64_t)O * I;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t oi = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; oi < total; oi += warps) {
        const int o = (int)(oi / I), i = (int)(oi - (int64_t)o * I);
        const T* p0 = partial + (size_t)o * ldo;
        const T sc = scaler ? scaler[oi] : T(1);
        T gs = T(0);
        const int last = gbw ? R : R - 1;
        for (int r = (gsw || gscaler) ? 0 : R; r <= last; ++r) {
            const T* src = p0 + (r < R ? (size_t)i * sI + r : (size_t)boff + (size_t)i * sB);
            T d = T(0);
            for (int s = lane; s < splits; s += 32) d += src[(size_t)s * split_stride];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
            if (r < R) {
                if (gsw && lane == 0) gsw[(size_t)oi * R + r] = scaler ? sc * d : d;
                if (gscaler) gs += sw[(size_t)oi * R + r] * d;
            } else if (lane == 0) {
                gbw[oi] = d;
            }
        }
        if (gscaler && lane == 0) gscaler[oi] = gs;
    }
}

// ---------------------------------------------------------------------------
// Backward, input:  gx[n,i] = sum_j der_j (sum_o dY[n,o] W_eff[o,i,s+j]) + silu'(x) sum_o dY[n,o] bw[o,i]
// ---------------------------------------------------------------------------
constexpr int BI_TN = 32, BI_TI = 8, BI_THREADS = 256;

template <typename T, int K>
__global__ void __launch_bounds__(BI_THREADS)
bwd_input_simt_kernel(const T* __restrict__ dY, const T* __restrict__ x, const T* __restrict__ grid,
                      const T* __restrict__ bw, const T* __restrict__ sw, const T* __restrict__ scaler,
                      T* __restrict__ gx, int64_t N, int I, int O, int G, int CO) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = G + K, nk = G + 2 * K + 1, RW = R + 1;
    T* Wt = reinterpret_cast<T*>(smem_raw);          // [CO][TI][RW]
    T* dYs = Wt + (size_t)CO * BI_TI * RW;           // [TN][CO]
    T* knots = dYs + (size_t)BI_TN * CO;             // [TI][nk]
    const int tid = threadIdx.x;
    const int ti = tid & (BI_TI - 1), tn = tid / BI_TI;
    const int i0 = blockIdx.y * BI_TI;
    const int64_t n0 = (int64_t)blockIdx.x * BI_TN;
    const int i = i0 + ti;
    const int64_t n = n0 + tn;
    const bool live = (i < I) && (n < N);

    for (int e = tid; e < BI_TI * nk; e += BI_THREADS) {
        const int ii = e / nk, q = e - ii * nk;
        knots[e] = (i0 + ii < I) ? grid[(size_t)(i0 + ii) * nk + q] : T(0);
    }
    __syncthreads();
    T dw[K + 1];
    int s = 0;
    T sg = T(0);
#pragma unroll
    for (int j = 0; j <= K; ++j) dw[j] = T(0);
    if (live) {
        const T xv = x[(size_t)n * I + i];
        const T* t = knots + (size_t)ti * nk;
        const int m = locate_span(t, nk, xv);
        if (m >= 0) {
            T v[K + 1], d[K + 1];
            window_values<K, T, true>(t, nk, m, xv, v, d);
            s = window_in_range<K, T>(m, R, d, dw);
        }
        if (bw) sg = silu_grad_t<T>(xv);
    }
    T acc[K + 1];
    T accb = T(0);
#pragma unroll
    for (int j = 0; j <= K; ++j) acc[j] = T(0);

    for (int oc = 0; oc < O; oc += CO) {
        const int co = (O - oc < CO) ? (O - oc) : CO;
        __syncthreads();
        for (int e = tid; e < co * BI_TI * R; e += BI_THREADS) {
            const int o = e / (BI_TI * R);
            const int rem = e - o * (BI_TI * R);
            const int ii = rem / R, r = rem - ii * R;
            T w = T(0);
            if (i0 + ii < I) {
                const size_t oi = (size_t)(oc + o) * I + i0 + ii;
                w = sw[oi * R + r];
                if (scaler) w *= scaler[oi];
            }
            Wt[((size_t)o * BI_TI + ii) * RW + r] = w;
        }
        for (int e = tid; e < co * BI_TI; e += BI_THREADS) {
            const int o = e / BI_TI, ii = e - o * BI_TI;
            Wt[((size_t)o * BI_TI + ii) * RW + R] =
                (bw && i0 + ii < I) ? bw[(size_t)(oc + o) * I + i0 + ii] : T(0);
        }
        for (int e = tid; e < BI_TN * co; e += BI_THREADS) {
            const int nn = e / co, o = e - nn * co;
            dYs[(size_t)nn * CO + o] = (n0 + nn < N) ? dY[(size_t)(n0 + nn) * O + oc + o] : T(0);
        }
        __syncthreads();
        const T* dyr = dYs + (size_t)tn * CO;
        for (int o = 0; o < co; ++o) {
            const T dy = dyr[o];
            const T* wp = Wt + ((size_t)o * BI_TI + ti) * RW;
#pragma unroll
            for (int j = 0; j <= K; ++j) acc[j] += dy * wp[s + j];
            accb += dy * wp[R];
        }
    }
    if (live) {
        T g = accb * sg;
#pragma unroll
        for (int j = 0; j <= K; ++j) g += acc[j] * dw[j];
        gx[(size_t)n * I + i] = g;
    }
}

inline int grid_1d(int64_t work, int threads, int cap = 148 * 32) {
    int64_t b = (work + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > cap) b = cap;
    return (int)b;
}

// Grid of the table-driven basis kernels: x = groups of 32 features, y = row ranges sized so that
// about 6 blocks per SM exist, with at least 64 rows each (a block copies 32 KB of tables first).
inline void basis_table_grid(const LayerShape& s, dim3& g, int64_t& rows_per_block) {
    const int fgroups = (s.I + BT_FEATURES - 1) / BT_FEATURES;
    int64_t ry = (148 * 6 + fgroups - 1) / fgroups;
    const int64_t max_ry = (s.N + 63) / 64;
    if (ry > max_ry) ry = max_ry;
    if (ry < 1) ry = 1;
    if (ry > 65535) ry = 65535;
    rows_per_block = (s.N + ry - 1) / ry;
    g = dim3((unsigned)fgroups, (unsigned)((s.N + rows_per_block - 1) / rows_per_block));
}

#define KAN_DISPATCH_K(Kval, ...)                                   \
    switch (Kval) {                                                 \
        case 1: { constexpr int KK = 1; __VA_ARGS__; break; }       \
        case 2: { constexpr int KK = 2; __VA_ARGS__; break; }       \
        default: { constexpr int KK = 3; __VA_ARGS__; break; }      \
    }

template <typename T>
struct ParamPlan {
    int rmax, opt, tns, to, splits;
    int64_t n_per_split;
};

template <typename T>
ParamPlan<T> plan_param(const LayerShape& s) {
    ParamPlan<T> p;
    const int R = s.R();
    p.rmax = R <= 8 ? 8 : (R <= 16 ? 16 : (R <= 32 ? 32 : 72));
    p.opt = p.rmax <= 16 ? 4 : 1;
    p.tns = p.rmax >= 32 ? 8 : (p.rmax == 16 ? 16 : 32);
    p.to = 32 * p.opt;
    const int64_t bxy = (int64_t)((s.O + p.to - 1) / p.to) * ((s.I + BP_TI - 1) / BP_TI);
    int64_t splits = (4 * 148 + bxy - 1) / bxy;
    const int64_t max_splits = (s.N + 63) / 64;
    if (splits > max_splits) splits = max_splits;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    p.n_per_split = (s.N + splits - 1) / splits;
    p.n_per_split = (p.n_per_split + p.tns - 1) / p.tns * p.tns;
    if (p.n_per_split < p.tns) p.n_per_split = p.tns;          // empty batch: one (empty) split
    p.splits = (int)((s.N + p.n_per_split - 1) / p.n_per_split);
    if (p.splits < 1) p.splits = 1;
    return p;
}

template <typename T, int K>
cudaError_t launch_bwd_param(const ParamPlan<T>& p, const T* dY, const T* x, const T* grid, T* partial,
                             const LayerShape& s, bool has_base, cudaStream_t st) {
    dim3 g((s.O + p.to - 1) / p.to, (s.I + BP_TI - 1) / BP_TI, p.splits);
#define KAN_BP(RM, OP, TN)                                                                     \
    bwd_param_simt_kernel<T, K, RM, OP, TN><<<g, BP_THREADS, 0, st>>>(dY, x, grid, partial, s.N, s.I, s.O, \
                                                                      s.G, has_base, p.n_per_split)
    if (p.rmax == 8) KAN_BP(8, 4, 32);
    else if (p.rmax == 16) KAN_BP(16, 4, 16);
    else if (p.rmax == 32) KAN_BP(32, 1, 8);
    else KAN_BP(72, 1, 8);
#undef KAN_BP
    return cudaGetLastError();
}

}  // namespace

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
template <typename T>
cudaError_t simt_basis(const T* x, const T* grid, T* H, const LayerShape& s, cudaStream_t st) {
    const int64_t pairs = s.N * s.I;
    if (pairs == 0) return cudaSuccess;
    const int R = s.R();
    if (sizeof(T) == 4 && R == 8 && s.T() <= 13 && (reinterpret_cast<uintptr_t>(H) & 15) == 0) {
        const int blocks = grid_1d((pairs + 31) / 32, 8, 148 * 8);
        KAN_DISPATCH_K(s.K, (basis_r8_kernel<KK><<<blocks, 256, 0, st>>>(
                                 reinterpret_cast<const float*>(x), reinterpret_cast<const float*>(grid),
                                 reinterpret_cast<float*>(H), pairs, s.I, s.G)));
        return cudaGetLastError();
    }
    int P = 128;
    while (P > 32 && (size_t)P * R * sizeof(T) > 40 * 1024) P >>= 1;
    const size_t smem = (size_t)P * R * sizeof(T);
    const int blocks = grid_1d(pairs, P, 148 * 16);
    KAN_DISPATCH_K(s.K, (basis_kernel<T, KK><<<blocks, P, smem, st>>>(x, grid, H, pairs, s.I, s.G)));
    return cudaGetLastError();
}

template <typename T>
cudaError_t simt_basis_grad(const T* x, const T* grid, const T* gH, T* gx, const LayerShape& s, cudaStream_t st) {
    const int64_t pairs = s.N * s.I;
    if (pairs == 0) return cudaSuccess;
    const int blocks = grid_1d(pairs, 256);
    if (sizeof(T) == 4 && s.R() == 8 && (reinterpret_cast<uintptr_t>(gH) & 15) == 0) {
        KAN_DISPATCH_K(s.K, (basis_grad_r8_kernel<KK><<<blocks, 256, 0, st>>>(
                                 reinterpret_cast<const float*>(x), reinterpret_cast<const float*>(grid),
                                 reinterpret_cast<const float*>(gH), reinterpret_cast<float*>(gx), pairs, s.I, s.G)));
        return cudaGetLastError();
    }
    KAN_DISPATCH_K(s.K, (basis_grad_kernel<T, KK><<<blocks, 256, 0, st>>>(x, grid, gH, gx, pairs, s.I, s.G)));
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Forward for up to 255 rows (small batches; larger float32 batches take the tensor-core path):
// the weights are the traffic, so they are streamed exactly once per block of 8 rows (measured
// against the tiled kernel below, which restages every weight tile per 32 rows: 256 -> 256 at 255
// rows 0.09 vs 0.34 ms, 64 -> 64 with G = 64 0.03 vs 0.48 ms).  A block = 8 warps = 8 outputs x 8 rows;
// the basis windows of the rows are staged in shared memory per chunk of 128 features, then
// lane = feature: each lane reads the k+1 weights of its window (consecutive lanes read
// consecutive weight rows) and the warp reduces over the features by shuffles.
// ---------------------------------------------------------------------------
constexpr int FR_THREADS = 256, FR_NR = 8, FR_IC = 128, FR_MAX_ROWS = 255;

template <typename T, int K>
__global__ void __launch_bounds__(FR_THREADS)
fwd_rows_kernel(const T* __restrict__ x, const T* __restrict__ grid, const T* __restrict__ bw,
                const T* __restrict__ sw, const T* __restrict__ scaler, T* __restrict__ y,
                int64_t N, int I, int O, int G) {
    __shared__ T vals[FR_NR][FR_IC][K + 1];
    __shared__ T sil[FR_NR][FR_IC];
    __shared__ int st[FR_NR][FR_IC];
    const int R = G + K, nk = G + 2 * K + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int o = blockIdx.x * (FR_THREADS / 32) + warp;
    const int64_t n0 = (int64_t)blockIdx.y * FR_NR;
    T acc[FR_NR];
#pragma unroll
    for (int n = 0; n < FR_NR; ++n) acc[n] = T(0);

    for (int i0 = 0; i0 < I; i0 += FR_IC) {
        const int ic = (I - i0 < FR_IC) ? (I - i0) : FR_IC;
        __syncthreads();
        for (int e = tid; e < FR_NR * ic; e += FR_THREADS) {
            const int n = e / ic, i = e - n * ic;
            T w[K + 1];
            int s = 0;
            T sv = T(0);
#pragma unroll
            for (int j = 0; j <= K; ++j) w[j] = T(0);
            if (n0 + n < N) {
                const T xv = x[(size_t)(n0 + n) * I + (i0 + i)];
                const T* t = grid + (size_t)(i0 + i) * nk;
                const int m = locate_span(t, nk, xv);
                if (m >= 0) {
                    T v[K + 1], d[K + 1];
                    window_values<K, T, false>(t, nk, m, xv, v, d);
                    s = window_in_range<K, T>(m, R, v, w);
                }
                sv = bw ? silu_t<T>(xv) : T(0);
            }
#pragma unroll
            for (int j = 0; j <= K; ++j) vals[n][i][j] = w[j];
            sil[n][i] = sv;
            st[n][i] = s;
        }
        __syncthreads();
        if (o < O) {
            for (int i = lane; i < ic; i += 32) {
                const size_t oi = (size_t)o * I + (i0 + i);
                const T* wrow = sw + oi * R;
                const T sc = scaler ? scaler[oi] : T(1);
                const T b = bw ? bw[oi] : T(0);
#pragma unroll
                for (int n = 0; n < FR_NR; ++n) {
                    const int s = st[n][i];
                    T dot = T(0);
#pragma unroll
                    for (int j = 0; j <= K; ++j) dot += vals[n][i][j] * wrow[s + j];
                    acc[n] += sc * dot + sil[n][i] * b;
                }
            }
        }
    }
#pragma unroll
    for (int n = 0; n < FR_NR; ++n) {
        T v = acc[n];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0 && o < O && n0 + n < N) y[(size_t)(n0 + n) * O + o] = v;
    }
}

bool basis_table_supported(const LayerShape& s) {
    // below about two million values the extra launch of the table kernel costs more than it saves
    return s.R() == 8 && s.T() <= 12 && s.K >= 1 && s.K <= 3 && s.N >= 256 && s.N * s.I >= (int64_t)1 << 21;
}

cudaError_t simt_basis_table(const float* x, const float* tab, int fs, float* H, const LayerShape& s,
                             cudaStream_t st) {
    dim3 g;
    int64_t rows_per_block;
    basis_table_grid(s, g, rows_per_block);
    basis_table_kernel<<<g, BT_THREADS, 0, st>>>(x, tab, fs, H, s.N, s.I, s.G, s.K, rows_per_block);
    return cudaGetLastError();
}

cudaError_t simt_basis_grad_table(const float* x, const float* tab, int fs, const float* gH, float* gx,
                                  const LayerShape& s, cudaStream_t st) {
    dim3 g;
    int64_t rows_per_block;
    basis_table_grid(s, g, rows_per_block);
    basis_grad_table_kernel<<<g, BT_THREADS, 0, st>>>(x, tab, fs, gH, gx, s.N, s.I, s.G, s.K, rows_per_block);
    return cudaGetLastError();
}

template <typename T>
cudaError_t simt_forward(const T* x, const T* grid, const T* bw, const T* sw, const T* scaler, T* y,
                         const LayerShape& s, cudaStream_t st) {
    if (s.N == 0) return cudaSuccess;
    if (s.N <= FR_MAX_ROWS) {
        dim3 g((s.O + FR_THREADS / 32 - 1) / (FR_THREADS / 32), (unsigned)((s.N + FR_NR - 1) / FR_NR));
        KAN_DISPATCH_K(s.K, (fwd_rows_kernel<T, KK><<<g, FR_THREADS, 0, st>>>(x, grid, bw, sw, scaler, y, s.N, s.I,
                                                                              s.O, s.G)));
        return cudaGetLastError();
    }
    const int RW = s.R() + 1;
    int CI = (int)(32768 / ((size_t)RW * (FW_TO + 1) * sizeof(T)));
    if (CI > 16) CI = 16;
    if (CI > s.I) CI = s.I;
    if (CI < 1) CI = 1;
    FwdSmem<T> L{CI, RW, s.K + 1, s.T()};
    const size_t smem = L.bytes();
    dim3 g((unsigned)((s.N + FW_TN - 1) / FW_TN), (s.O + FW_TO - 1) / FW_TO);
    if (g.y > 65535u) return cudaErrorInvalidConfiguration;
    cudaError_t e = cudaSuccess;
    KAN_DISPATCH_K(s.K, {
        if (smem > 48 * 1024)
            e = cudaFuncSetAttribute(fwd_simt_kernel<T, KK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            fwd_simt_kernel<T, KK><<<g, FW_THREADS, smem, st>>>(x, grid, bw, sw, scaler, y, s.N, s.I, s.O, s.G, CI);
    });
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

template <typename T>
size_t simt_backward_workspace(const LayerShape& s, bool need_param) {
    if (!need_param) return 0;
    ParamPlan<T> p = plan_param<T>(s);
    return (size_t)p.splits * s.O * s.I * (s.R() + 1) * sizeof(T);
}

template <typename T>
cudaError_t finalize_param_grads(const T* partial, int splits, int64_t split_stride,
                                 int64_t ldo, int sI, int64_t boff, int sB,
                                 const T* sw, const T* scaler, T* gsw, T* gscaler, T* gbw,
                                 int O, int I, int R, cudaStream_t st) {
    if (splits >= 8) {
        const int blocks = grid_1d((int64_t)O * I * 32, 256);
        finalize_param_wide_kernel<T><<<blocks, 256, 0, st>>>(partial, splits, split_stride, ldo, sI, boff, sB,
                                                             sw, scaler, gsw, gscaler, gbw, O, I, R);
        return cudaGetLastError();
    }
    const int blocks = grid_1d((int64_t)O * I, 128);
    finalize_param_kernel<T><<<blocks, 128, 0, st>>>(partial, splits, split_stride, ldo, sI, boff, sB,
                                                    sw, scaler, gsw, gscaler, gbw, O, I, R);
    return cudaGetLastError();
}

template <typename T>
cudaError_t simt_backward(const T* dY, const T* x, const T* grid, const T* bw, const T* sw, const T* scaler,
                          T* gx, T* gbw, T* gsw, T* gscaler, const LayerShape& s,
                          void* ws, size_t ws_bytes, cudaStream_t st) {
    if (s.N == 0) {
        // Sums over an empty batch are zero.
        cudaError_t e = cudaSuccess;
        const size_t oi = (size_t)s.O * s.I;
        if (gbw) e = cudaMemsetAsync(gbw, 0, oi * sizeof(T), st);
        if (e == cudaSuccess && gsw) e = cudaMemsetAsync(gsw, 0, oi * s.R() * sizeof(T), st);
        if (e == cudaSuccess && gscaler) e = cudaMemsetAsync(gscaler, 0, oi * sizeof(T), st);
        return e;
    }
    cudaError_t e = cudaSuccess;
    const bool need_param = gbw || gsw || gscaler;
    if (need_param) {
        ParamPlan<T> p = plan_param<T>(s);
        const size_t need = (size_t)p.splits * s.O * s.I * (s.R() + 1) * sizeof(T);
        if (!ws || ws_bytes < need) return cudaErrorMemoryAllocation;
        T* partial = reinterpret_cast<T*>(ws);
        KAN_DISPATCH_K(s.K, (e = launch_bwd_param<T, KK>(p, dY, x, grid, partial, s, bw != nullptr, st)));
        if (e != cudaSuccess) return e;
        const int RW = s.R() + 1;
        e = finalize_param_grads<T>(partial, p.splits, (int64_t)s.O * s.I * RW, (int64_t)s.I * RW, RW,
                                    s.R(), RW, sw, scaler, gsw, gscaler, bw ? gbw : nullptr,
                                    s.O, s.I, s.R(), st);
        if (e != cudaSuccess) return e;
    }
    if (gx) {
        const int RW = s.R() + 1;
        int CO = (int)(32768 / ((size_t)BI_TI * RW * sizeof(T)));
        if (CO > 64) CO = 64;
        if (CO > s.O) CO = s.O;
        if (CO < 1) CO = 1;
        const size_t smem = ((size_t)CO * BI_TI * RW + (size_t)BI_TN * CO + (size_t)BI_TI * s.T()) * sizeof(T);
        dim3 g((unsigned)((s.N + BI_TN - 1) / BI_TN), (s.I + BI_TI - 1) / BI_TI);
        if (g.y > 65535u) return cudaErrorInvalidConfiguration;
        KAN_DISPATCH_K(s.K, {
            if (smem > 48 * 1024)
                e = cudaFuncSetAttribute(bwd_input_simt_kernel<T, KK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                bwd_input_simt_kernel<T, KK><<<g, BI_THREADS, smem, st>>>(dY, x, grid, bw, sw, scaler, gx,
                                                                         s.N, s.I, s.O, s.G, CO);
        });
        if (e != cudaSuccess) return e;
        e = cudaGetLastError();
    }
    return e;
}

#define KAN_INSTANTIATE(T)                                                                                      \
    template cudaError_t simt_basis<T>(const T*, const T*, T*, const LayerShape&, cudaStream_t);               \
    template cudaError_t simt_basis_grad<T>(const T*, const T*, const T*, T*, const LayerShape&, cudaStream_t); \
    template cudaError_t simt_forward<T>(const T*, const T*, const T*, const T*, const T*, T*,                 \
                                         const LayerShape&, cudaStream_t);                                     \
    template size_t simt_backward_workspace<T>(const LayerShape&, bool);                                       \
    template cudaError_t finalize_param_grads<T>(const T*, int, int64_t, int64_t, int, int64_t, int,           \
                                                 const T*, const T*, T*, T*, T*, int, int, int, cudaStream_t); \
    template cudaError_t simt_backward<T>(const T*, const T*, const T*, const T*, const T*, const T*,          \
                                          T*, T*, T*, T*, const LayerShape&, void*, size_t, cudaStream_t);
KAN_INSTANTIATE(float)
KAN_INSTANTIATE(double)

}  // namespace kanb200
