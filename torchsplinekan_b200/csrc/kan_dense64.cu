// Float64 layer kernels on the FP64 matrix instruction (mma.sync m8n8k4; tcgen05 has no FP64
// kind).  Measured on the part: 36.8 TFLOP/s for a register-only loop of that instruction against
// 31.0 TFLOP/s for the FMA pipe, and -- what matters more here -- one instruction per 256 FMAs, so
// the issue slots stay free for the threads that evaluate the basis functions.
//
// All three kernels use the DENSE formulation of the layer (reference: spline_kan/
// reference_backend.py:96-125, csrc/kan_cuda.cu:469-630): with RW = R + 1 columns per input feature
// (R spline slots, then the SiLU value) and c = i RW + r,
//      forward            y[n, o]  = sum_c A[n, c] W[o, c]
//      parameter gradient D[o, c]  = sum_n dY[n, o] A[n, c]
//      input gradient     gx[n, i] = sum_r dA[n, i RW + r] (sum_o dY[n, o] W[o, c])
// where row n of A holds the k + 1 non-zero basis values of every feature (zeros elsewhere) and
// dA their x-derivatives (SiLU' in the last slot).  A and dA tiles are evaluated from x into shared
// memory by all threads of the block, 64 rows x at most 96 columns at a time; the weight image
// W[o][c] (coefficients times scaler, base weight in the last slot) is written once per call by a
// small kernel.  Two blocks share an SM, so one block's evaluation phase overlaps the other's
// matrix phase.  Shared tiles have a leading dimension of 4 (mod 16) doubles, which makes both
// fragment access patterns of the instruction (row g, column t and row t, column g; lane = 4 g + t)
// conflict-free per half-warp.
//
// Sums over rows are per-split partial slabs reduced in a fixed order by finalize_param_grads: no
// atomics, bitwise reproducible.
#include "kan_device.cuh"
#include "kan_dmma.cuh"
#include "kan_internal.h"
#include "kan_tc_common.cuh"
#include "kan_tc_ptx.cuh"

namespace kanb200 {

namespace {
using namespace ptx;

constexpr int DM_THREADS = 256;
constexpr int DM_ROWS = 64;          // rows of x / dY per tile
constexpr int DM_CK = 96;            // columns of A per chunk (forward, parameter gradient)
constexpr int DM_CK_DX = 64;         // columns per chunk of the input-gradient kernel
constexpr int DM_KO = 64;            // outputs per reduction chunk of the input-gradient kernel
constexpr int DM_MIN_ROWS = 512;

__host__ __device__ inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
__host__ __device__ inline int lead_dim(int cols) { return round_up(cols, 16) + 4; }

__global__ void dm_pack_weights_kernel(const double* __restrict__ sw, const double* __restrict__ scaler,
                                       const double* __restrict__ bw, double* __restrict__ Wimg,
                                       int O, int I, int R) {
    const int RW = R + 1;
    const int64_t pairs = (int64_t)O * I;
    for (int64_t oi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; oi < pairs;
         oi += (int64_t)gridDim.x * blockDim.x) {
        const double sc = scaler ? scaler[oi] : 1.0;
        double* out = Wimg + oi * RW;
        for (int r = 0; r < R; ++r) out[r] = sw[oi * R + r] * sc;
        out[R] = bw ? bw[oi] : 0.0;
    }
}

// Reciprocal knot differences of one feature, rc[(d - 1) nk + j] = 1 / (t[j + d] - t[j]) (0 where the
// knots coincide or j + d runs past the end): the six FP64 divisions of a cubic window become
// multiplications (a division costs about as much as the rest of the window).  A product with a
// rounded reciprocal differs from the quotient by at most one ulp.
__device__ __forceinline__ void load_knots(double* __restrict__ knots, const double* __restrict__ grid_rows, int ci,
                                           int CI, int nk, int K) {
    for (int e = threadIdx.x; e < ci * nk; e += DM_THREADS) knots[e] = grid_rows[e];
    double* rc = knots + (size_t)CI * nk;
    for (int e = threadIdx.x; e < ci * K * nk; e += DM_THREADS) {
        const int i = e / (K * nk), rem = e - i * (K * nk);
        const int d = rem / nk + 1, j = rem - (d - 1) * nk;
        double v = 0.0;
        if (j + d < nk) {
            const double width = grid_rows[(size_t)i * nk + j + d] - grid_rows[(size_t)i * nk + j];
            if (width != 0.0) v = 1.0 / width;
        }
        rc[e] = v;
    }
}

// window_values of kan_device.cuh with the divisions taken from the table above.  Reads at
// clamped positions (spans next to either end of the knot vector) only reach window slots whose
// basis index lies outside [0, R), which the caller drops.
template <int K, bool DERIV>
__device__ __forceinline__ void window_values_rc(const double* __restrict__ t, const double* __restrict__ rc, int nk,
                                                 int m, double x, double (&val)[K + 1], double (&der)[K + 1]) {
    double kn[2 * K];
#pragma unroll
    for (int e = 0; e < 2 * K; ++e) {
        int at = m - K + 1 + e;
        at = at < 0 ? 0 : (at > nk - 1 ? nk - 1 : at);
        kn[e] = t[at];
    }
    double b[K + 1];
    b[0] = 1.0;
#pragma unroll
    for (int j = 1; j <= K; ++j) b[j] = 0.0;
#pragma unroll
    for (int d = 1; d <= K; ++d) {
        double q[K + 1];
#pragma unroll
        for (int j = 0; j < d; ++j) {
            int at = m + 1 + j - d;
            at = at < 0 ? 0 : (at > nk - 1 - d ? nk - 1 - d : at);
            q[j] = b[j] * rc[(d - 1) * nk + at];
        }
        if (DERIV && d == K) {
#pragma unroll
            for (int j = 0; j <= K; ++j)
                der[j] = double(K) * ((j > 0 ? q[j - 1] : 0.0) - (j < K ? q[j] : 0.0));
        }
#pragma unroll
        for (int j = d; j >= 0; --j) {
            const double rising = (j > 0) ? (x - kn[K - 1 - d + j]) * q[j - 1] : 0.0;
            const double falling = (j < d) ? (kn[K + j] - x) * q[j] : 0.0;
            b[j] = rising + falling;
        }
    }
#pragma unroll
    for (int j = 0; j <= K; ++j) val[j] = b[j];
}

// The non-zero entries of one row piece of A (DERIV = false) or dA (DERIV = true): the k + 1 window
// values of one (sample, feature) and the SiLU slot.  The piece was zero-filled before.
template <int K, bool DERIV>
__device__ __forceinline__ void fill_piece(double* __restrict__ row, const double* __restrict__ t,
                                           const double* __restrict__ rc, int nk, int R, double xv, bool has_base) {
    const int m = locate_span(t, nk, xv);
    if (m >= 0) {
        double v[K + 1], d[K + 1];
        window_values_rc<K, DERIV>(t, rc, nk, m, xv, v, d);
#pragma unroll
        for (int j = 0; j <= K; ++j) {
            const int r = m - K + j;
            if (r >= 0 && r < R) row[r] = DERIV ? d[j] : v[j];
        }
    }
    if (has_base) row[R] = DERIV ? silu_grad_t<double>(xv) : silu_t<double>(xv);
}

// Zero-fills `doubles` (even) consecutive doubles of shared memory, 16 bytes per store.
__device__ __forceinline__ void zero_tile(double* __restrict__ tile, int doubles) {
    double2* t2 = reinterpret_cast<double2*>(tile);
    const int n2 = doubles >> 1;
#pragma unroll 4
    for (int e = threadIdx.x; e < n2; e += DM_THREADS) t2[e] = make_double2(0.0, 0.0);
}

// Evaluates the tile of A / dA for rows [r0, r0 + 64) and features [i0, i0 + ci) into a zero-filled
// tile.  `knots` holds the knot rows of the chunk, then their reciprocal tables.  Two pieces per
// iteration: their dependent chains (span search, recurrence, exp) interleave.
template <int K, bool DERIV>
__device__ __forceinline__ void fill_tile(double* __restrict__ As, int ld, const double* __restrict__ knots,
                                          const double* __restrict__ x, int64_t r0, int64_t r_end, int I, int i0,
                                          int ci, int CI, int nk, int R, bool has_base) {
    const int RW = R + 1, total = DM_ROWS * ci;
    const double* rc = knots + CI * nk;
    const double* xrow = x + (size_t)r0 * I + i0;
    const int rows = (r_end - r0 < DM_ROWS) ? (int)(r_end - r0) : DM_ROWS;
    for (int p = threadIdx.x; p < total; p += 2 * DM_THREADS) {
        const int p2 = p + DM_THREADS;
        const int n = p / ci, i = p - n * ci;
        const int n2 = p2 / ci, i2 = p2 - n2 * ci;
        const bool live = n < rows, live2 = p2 < total && n2 < rows;
        const double xv = live ? xrow[(size_t)n * I + i] : 0.0;
        const double xv2 = live2 ? xrow[(size_t)n2 * I + i2] : 0.0;
        if (live) fill_piece<K, DERIV>(As + n * ld + i * RW, knots + i * nk, rc + i * K * nk, nk, R, xv, has_base);
        if (live2)
            fill_piece<K, DERIV>(As + n2 * ld + i2 * RW, knots + i2 * nk, rc + i2 * K * nk, nk, R, xv2, has_base);
    }
}

// Copies rows [0, nrows) x columns [0, ncols) of a row-major global matrix (leading dimension lds)
// into a shared tile, zero beyond (rows_live, cols_live); one warp per row, 16 bytes per lane where
// the addresses allow.
__device__ __forceinline__ void load_tile(double* __restrict__ dst, int ldd, const double* __restrict__ src,
                                          size_t lds, int nrows, int ncols, int rows_live, int cols_live) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool vec = ((lds | (size_t)cols_live) & 1) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                     (ncols & 1) == 0;
    for (int r = warp; r < nrows; r += DM_THREADS / 32) {
        const double* s = src + (size_t)r * lds;
        double* d = dst + r * ldd;
        const bool live = r < rows_live;
        if (vec) {
            for (int c = 2 * lane; c < ncols; c += 64) {
                double2 v = make_double2(0.0, 0.0);
                if (live && c < cols_live) v = *reinterpret_cast<const double2*>(s + c);
                *reinterpret_cast<double2*>(d + c) = v;
            }
        } else {
            for (int c = lane; c < ncols; c += 32) d[c] = (live && c < cols_live) ? s[c] : 0.0;
        }
    }
}

// The same copy by the bulk-copy engine, so that it runs while the block evaluates basis functions:
// warp 0 issues one copy per live row, completion (bytes) on `bar`; the other threads zero the
// ragged edges.  Needs 16-byte aligned rows and an even number of live columns (bulk_rows_ok).
struct TileCopy {
    double* dst;
    int ldd;
    const double* src;
    size_t lds;
    int nrows, ncols, rows_live, cols_live;
    __device__ __forceinline__ bool bulk_ok() const {
        return ((lds | (size_t)cols_live | (size_t)ldd) & 1) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    }
    __device__ __forceinline__ int live_rows() const { return rows_live < nrows ? (rows_live < 0 ? 0 : rows_live) : nrows; }
    __device__ __forceinline__ int live_cols() const { return cols_live < ncols ? cols_live : ncols; }
    __device__ __forceinline__ uint32_t bytes() const { return (uint32_t)live_rows() * (uint32_t)live_cols() * 8u; }
    __device__ __forceinline__ void issue(uint32_t bar) const {        // warp 0, after expect_tx
        const int lane = threadIdx.x & 31, lr = live_rows();
        const uint32_t row_bytes = (uint32_t)live_cols() * 8u;
        if (row_bytes == 0) return;
        for (int r = lane; r < lr; r += 32) bulk_g2s(smem_u32(dst + r * ldd), src + (size_t)r * lds, row_bytes, bar);
    }
    __device__ __forceinline__ void zero_edges() const {               // all threads
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, lr = live_rows(), lc = live_cols();
        for (int r = warp; r < nrows; r += DM_THREADS / 32)
            for (int c = (r < lr ? lc : 0) + lane; c < ncols; c += 32) dst[r * ldd + c] = 0.0;
    }
    __device__ __forceinline__ void by_threads() const {
        load_tile(dst, ldd, src, lds, nrows, ncols, rows_live, cols_live);
    }
};

// Starts up to two tile copies; returns true when they went to the bulk-copy engine (the caller
// then waits on `bar` before reading the tiles).
__device__ __forceinline__ bool start_copies(const TileCopy* a, const TileCopy* b, uint32_t bar) {
    const bool bulk = a->bulk_ok() && (b == nullptr || b->bulk_ok());
    if (!bulk) {
        a->by_threads();
        if (b) b->by_threads();
        return false;
    }
    if (threadIdx.x < 32) {
        if (threadIdx.x == 0) mbar_arrive_expect_tx(bar, a->bytes() + (b ? b->bytes() : 0u));
        __syncwarp();
        a->issue(bar);
        if (b) b->issue(bar);
    }
    a->zero_edges();
    if (b) b->zero_edges();
    return true;
}

struct BlockSync {
    uint64_t bar;
    int abort_flag;
};

__device__ __forceinline__ void block_sync_init(BlockSync* bs) {
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bs->bar), 1);
        bs->abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------
// forward: block = 64 rows x TO outputs, 8 warps as MW x NW, warp tile (8 WMT) x (8 WNT)
// ---------------------------------------------------------------------------
template <int K, int MW, int NW, int WMT, int WNT>
__global__ void __launch_bounds__(DM_THREADS, 2)
dm_forward_kernel(const double* __restrict__ x, const double* __restrict__ grid, const double* __restrict__ Wimg,
                  double* __restrict__ y, int64_t N, int I, int O, int G, int CI, bool has_base,
                  int* __restrict__ status) {
    constexpr int TO = NW * WNT * 8;
    static_assert(MW * NW * 32 == DM_THREADS && MW * WMT * 8 == DM_ROWS, "tile shape");
    extern __shared__ __align__(16) double dsm[];
    __shared__ BlockSync bs;
    block_sync_init(&bs);
    uint32_t phase = 0;
    const int R = G + K, RW = R + 1, nk = G + 2 * K + 1, ctot = I * RW;
    const int ld = lead_dim(round_up(CI * RW, 4));
    double* As = dsm;                          // [64][ld]
    double* Ws = As + (size_t)DM_ROWS * ld;    // [TO][ld]
    double* knots = Ws + (size_t)TO * ld;      // [CI][nk] knots, [CI][K][nk] reciprocals
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp % MW) * WMT * 8, n0 = (warp / MW) * WNT * 8;
    const int o0 = blockIdx.y * TO;
    const int nchunks = (I + CI - 1) / CI;
    const int64_t ntiles = (N + DM_ROWS - 1) / DM_ROWS;
    bool resident = false;                     // a single chunk's weights and knots stay in place

    for (int64_t rt = blockIdx.x; rt < ntiles; rt += gridDim.x) {
        const int64_t r0 = rt * DM_ROWS;
        double acc[WMT][WNT][2];
#pragma unroll
        for (int a = 0; a < WMT; ++a)
#pragma unroll
            for (int b = 0; b < WNT; ++b) acc[a][b][0] = acc[a][b][1] = 0.0;
        for (int ch = 0; ch < nchunks; ++ch) {
            const int i0 = ch * CI, ci = (I - i0 < CI) ? (I - i0) : CI;
            const int ck = ci * RW, ckp = round_up(ck, 4);
            __syncthreads();
            zero_tile(As, DM_ROWS * ld);
            bool pending = false;
            if (!resident) {
                load_knots(knots, grid + (size_t)i0 * nk, ci, CI, nk, K);
                const TileCopy w{Ws, ld, Wimg + (size_t)o0 * ctot + (size_t)i0 * RW, (size_t)ctot, TO, ckp, O - o0, ck};
                pending = start_copies(&w, nullptr, smem_u32(&bs.bar));
                resident = nchunks == 1;
            }
            __syncthreads();
            fill_tile<K, false>(As, ld, knots, x, r0, N, I, i0, ci, CI, nk, R, has_base);
            if (pending) {
                mbar_wait(smem_u32(&bs.bar), phase, &bs.abort_flag);
                phase ^= 1u;
            }
            __syncthreads();
            if (bs.abort_flag) {
                if (tid == 0) report_status(status, 3);
                return;
            }
            const double* ap = As + (m0 + g) * ld + t;
            const double* bp = Ws + (n0 + g) * ld + t;
            for (int k0 = 0; k0 < ckp; k0 += 4) {
                double a[WMT], b[WNT];
#pragma unroll
                for (int mt = 0; mt < WMT; ++mt) a[mt] = ap[mt * 8 * ld + k0];
#pragma unroll
                for (int nt = 0; nt < WNT; ++nt) b[nt] = bp[nt * 8 * ld + k0];
#pragma unroll
                for (int mt = 0; mt < WMT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < WNT; ++nt) dmma::m8n8k4(acc[mt][nt][0], acc[mt][nt][1], a[mt], b[nt]);
            }
        }
#pragma unroll
        for (int mt = 0; mt < WMT; ++mt) {
            const int64_t row = r0 + m0 + mt * 8 + g;
            if (row >= N) continue;
#pragma unroll
            for (int nt = 0; nt < WNT; ++nt) {
                const int col = o0 + n0 + nt * 8 + 2 * t;
                double* out = y + (size_t)row * O + col;
                if (col < O) out[0] = acc[mt][nt][0];
                if (col + 1 < O) out[1] = acc[mt][nt][1];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// parameter gradient: block = one group of CI features x TO outputs x one range of rows;
// M = columns of the group (up to 12 tiles of 8, dealt to the MW warp rows), N = outputs, K = rows
// ---------------------------------------------------------------------------
template <int K, int MW, int NW, int WNT>
__global__ void __launch_bounds__(DM_THREADS, 2)
dm_bwd_param_kernel(const double* __restrict__ dY, const double* __restrict__ x, const double* __restrict__ grid,
                    double* __restrict__ partial, int64_t N, int I, int O, int G, int CI, bool has_base,
                    int64_t n_per_split, int* __restrict__ status) {
    constexpr int TO = NW * WNT * 8;
    constexpr int QM = (DM_CK / 8 + MW - 1) / MW;
    static_assert(MW * NW * 32 == DM_THREADS, "tile shape");
    extern __shared__ __align__(16) double dsm[];
    __shared__ BlockSync bs;
    block_sync_init(&bs);
    uint32_t phase = 0;
    const int R = G + K, RW = R + 1, nk = G + 2 * K + 1, ctot = I * RW;
    const int lda = lead_dim(round_up(CI * RW, 8)), ldy = lead_dim(TO);
    double* As = dsm;                            // [64][lda]
    double* dYs = As + (size_t)DM_ROWS * lda;    // [64][ldy]
    double* knots = dYs + (size_t)DM_ROWS * ldy; // [CI][nk] knots, [CI][K][nk] reciprocals
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp % MW, n0 = (warp / MW) * WNT * 8;
    const int i0 = blockIdx.x * CI, ci = (I - i0 < CI) ? (I - i0) : CI;
    const int ck = ci * RW, ckp = round_up(ck, 8), mtiles = ckp / 8;
    const int o0 = blockIdx.z * TO;
    const int64_t nb = (int64_t)blockIdx.y * n_per_split;
    const int64_t ne = (nb + n_per_split < N) ? nb + n_per_split : N;

    load_knots(knots, grid + (size_t)i0 * nk, ci, CI, nk, K);
    double acc[QM][WNT][2];
#pragma unroll
    for (int q = 0; q < QM; ++q)
#pragma unroll
        for (int b = 0; b < WNT; ++b) acc[q][b][0] = acc[q][b][1] = 0.0;

    for (int64_t r0 = nb; r0 < ne; r0 += DM_ROWS) {
        __syncthreads();
        zero_tile(As, DM_ROWS * lda);
        const TileCopy d{dYs, ldy, dY + (size_t)r0 * O + o0, (size_t)O, DM_ROWS, TO,
                         (int)(ne - r0 < DM_ROWS ? ne - r0 : DM_ROWS), O - o0};
        const bool pending = start_copies(&d, nullptr, smem_u32(&bs.bar));
        __syncthreads();
        fill_tile<K, false>(As, lda, knots, x, r0, ne, I, i0, ci, CI, nk, R, has_base);
        if (pending) {
            mbar_wait(smem_u32(&bs.bar), phase, &bs.abort_flag);
            phase ^= 1u;
        }
        __syncthreads();
        if (bs.abort_flag) {
            if (tid == 0) report_status(status, 3);
            return;
        }
        const double* ap = As + t * lda + wm * 8 + g;
        const double* bp = dYs + t * ldy + n0 + g;
        for (int k0 = 0; k0 < DM_ROWS; k0 += 4) {
            double a[QM], b[WNT];
#pragma unroll
            for (int q = 0; q < QM; ++q) a[q] = (wm + MW * q < mtiles) ? ap[k0 * lda + MW * q * 8] : 0.0;
#pragma unroll
            for (int nt = 0; nt < WNT; ++nt) b[nt] = bp[k0 * ldy + nt * 8];
#pragma unroll
            for (int q = 0; q < QM; ++q) {
                if (wm + MW * q < mtiles) {
#pragma unroll
                    for (int nt = 0; nt < WNT; ++nt) dmma::m8n8k4(acc[q][nt][0], acc[q][nt][1], a[q], b[nt]);
                }
            }
        }
    }
    double* slab = partial + (size_t)blockIdx.y * O * ctot;
#pragma unroll
    for (int q = 0; q < QM; ++q) {
        const int c = (wm + MW * q) * 8 + g;
        if (c >= ck) continue;
#pragma unroll
        for (int nt = 0; nt < WNT; ++nt) {
            const int o = o0 + n0 + nt * 8 + 2 * t;
            if (o < O) slab[(size_t)o * ctot + (size_t)i0 * RW + c] = acc[q][nt][0];
            if (o + 1 < O) slab[(size_t)(o + 1) * ctot + (size_t)i0 * RW + c] = acc[q][nt][1];
        }
    }
}

// ---------------------------------------------------------------------------
// input gradient: block = 64 rows; per group of features  DW[64, ck] = dY[64, O] W[O, ck]  in
// chunks of 64 outputs, then the products  dA .* DW  replace dA in shared memory and one thread per
// (row, feature) adds up its RW entries.
// ---------------------------------------------------------------------------
template <int K>
__global__ void __launch_bounds__(DM_THREADS, 2)
dm_bwd_input_kernel(const double* __restrict__ dY, const double* __restrict__ x, const double* __restrict__ grid,
                    const double* __restrict__ Wimg, double* __restrict__ gx, int64_t N, int I, int O, int G,
                    int CI, bool has_base, int* __restrict__ status) {
    constexpr int MW = 2, WMT = 4, WNT = 2;      // 8 warps: 2 x 4, warp tile 32 rows x 16 columns
    extern __shared__ __align__(16) double dsm[];
    __shared__ BlockSync bs;
    block_sync_init(&bs);
    uint32_t phase = 0;
    const int R = G + K, RW = R + 1, nk = G + 2 * K + 1, ctot = I * RW;
    const int ldc = lead_dim(DM_CK_DX), ldy = lead_dim(DM_KO);
    double* dAs = dsm;                             // [64][ldc]
    double* Ws = dAs + (size_t)DM_ROWS * ldc;      // [64 outputs][ldc]
    double* dYs = Ws + (size_t)DM_KO * ldc;        // [64][ldy]
    double* knots = dYs + (size_t)DM_ROWS * ldy;   // [CI][nk] knots, [CI][K][nk] reciprocals
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp % MW) * WMT * 8, n0 = (warp / MW) * WNT * 8;
    const int nchunks = (I + CI - 1) / CI, nochunks = (O + DM_KO - 1) / DM_KO;
    const int64_t ntiles = (N + DM_ROWS - 1) / DM_ROWS;

    // gridDim.y == nchunks (layers of up to 64 outputs): the block owns one group of features and
    // keeps its weights and knots in shared memory for all of its row tiles
    const bool can_stay = nochunks == 1 && (int)gridDim.y >= nchunks;
    bool resident = false;

    for (int64_t rt = blockIdx.x; rt < ntiles; rt += gridDim.x) {
        const int64_t r0 = rt * DM_ROWS;
        for (int ch = blockIdx.y; ch < nchunks; ch += gridDim.y) {
            const int i0 = ch * CI, ci = (I - i0 < CI) ? (I - i0) : CI;
            const int ck = ci * RW, ckp = round_up(ck, 8);
            double acc[WMT][WNT][2];
#pragma unroll
            for (int a = 0; a < WMT; ++a)
#pragma unroll
                for (int b = 0; b < WNT; ++b) acc[a][b][0] = acc[a][b][1] = 0.0;
            for (int oc = 0; oc < nochunks; ++oc) {
                const int ob = oc * DM_KO, ko = (O - ob < DM_KO) ? (O - ob) : DM_KO, ko4 = round_up(ko, 4);
                __syncthreads();
                if (oc == 0) {
                    if (!resident) load_knots(knots, grid + (size_t)i0 * nk, ci, CI, nk, K);
                    zero_tile(dAs, DM_ROWS * ldc);
                }
                const TileCopy w{Ws, ldc, Wimg + (size_t)ob * ctot + (size_t)i0 * RW, (size_t)ctot, ko4, ckp, ko, ck};
                const TileCopy d{dYs, ldy, dY + (size_t)r0 * O + ob, (size_t)O, DM_ROWS, ko4,
                                 (int)(N - r0 < DM_ROWS ? N - r0 : DM_ROWS), ko};
                const bool need_d = nochunks > 1 || ch == (int)blockIdx.y;
                bool pending = false;
                if (!resident) pending = start_copies(&w, need_d ? &d : nullptr, smem_u32(&bs.bar));
                else if (need_d) pending = start_copies(&d, nullptr, smem_u32(&bs.bar));
                resident = can_stay;
                if (oc == 0) {
                    __syncthreads();
                    fill_tile<K, true>(dAs, ldc, knots, x, r0, N, I, i0, ci, CI, nk, R, has_base);
                }
                if (pending) {
                    mbar_wait(smem_u32(&bs.bar), phase, &bs.abort_flag);
                    phase ^= 1u;
                }
                __syncthreads();
                if (bs.abort_flag) {
                    if (tid == 0) report_status(status, 3);
                    return;
                }
                if (n0 < ckp) {
                    const double* ap = dYs + (m0 + g) * ldy + t;
                    const double* bp = Ws + t * ldc + n0 + g;
                    for (int k0 = 0; k0 < ko4; k0 += 4) {
                        double a[WMT], b[WNT];
#pragma unroll
                        for (int mt = 0; mt < WMT; ++mt) a[mt] = ap[mt * 8 * ldy + k0];
#pragma unroll
                        for (int nt = 0; nt < WNT; ++nt) b[nt] = bp[k0 * ldc + nt * 8];
#pragma unroll
                        for (int mt = 0; mt < WMT; ++mt)
#pragma unroll
                            for (int nt = 0; nt < WNT; ++nt)
                                dmma::m8n8k4(acc[mt][nt][0], acc[mt][nt][1], a[mt], b[nt]);
                    }
                }
            }
            // every (row, column) of the tile belongs to exactly one lane: multiply in place
#pragma unroll
            for (int mt = 0; mt < WMT; ++mt)
#pragma unroll
                for (int nt = 0; nt < WNT; ++nt) {
                    const int col = n0 + nt * 8 + 2 * t;
                    if (col < ckp) {
                        double2* p = reinterpret_cast<double2*>(dAs + (m0 + mt * 8 + g) * ldc + col);
                        double2 v = *p;
                        v.x *= acc[mt][nt][0];
                        v.y *= acc[mt][nt][1];
                        *p = v;
                    }
                }
            __syncthreads();
            for (int p = tid; p < DM_ROWS * ci; p += DM_THREADS) {
                const int n = p / ci, i = p - n * ci;
                if (r0 + n >= N) continue;
                // lanes of a warp start at different slots of their pieces: pieces that are 8 banks
                // apart would otherwise collide on every read
                const double* row = dAs + n * ldc + i * RW;
                double s = 0.0;
                int r = i % RW;
                for (int q = 0; q < RW; ++q) {
                    s += row[r];
                    r = (r + 1 == RW) ? 0 : r + 1;
                }
                gx[(size_t)(r0 + n) * I + i0 + i] = s;
            }
        }
    }
}

struct DmPlan {
    int ci, ci_dx;              // features per chunk
    int to;                     // outputs per block (64 or 8)
    int groups, otiles, splits;
    int64_t n_per_split;
    size_t w_bytes, slab_bytes; // weight image, one slab of partial sums
};

DmPlan dm_plan(const LayerShape& s) {
    DmPlan p;
    const int RW = s.R() + 1;
    p.ci = DM_CK / RW < 1 ? 1 : DM_CK / RW;
    p.ci_dx = DM_CK_DX / RW < 1 ? 1 : DM_CK_DX / RW;
    // 64 rows x a multiple of 4 features = whole passes of the block's 256 threads over the tile
    // (measured for the input gradient, 64 -> 64 and 64 -> 1 at 131072 rows: 4 features per chunk
    // 1.09 / 0.50 ms, 5 features 1.13 / 0.54 ms)
    if (p.ci >= 4) p.ci &= ~3;
    if (p.ci_dx >= 4) p.ci_dx &= ~3;
    if (p.ci > s.I) p.ci = s.I;
    if (p.ci_dx > s.I) p.ci_dx = s.I;
    p.to = s.O <= 8 ? 8 : 64;
    p.groups = (s.I + p.ci - 1) / p.ci;
    p.otiles = (s.O + p.to - 1) / p.to;
    int64_t splits = (2 * 148 + (int64_t)p.groups * p.otiles - 1) / ((int64_t)p.groups * p.otiles);
    const int64_t max_splits = (s.N + DM_ROWS - 1) / DM_ROWS;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    p.n_per_split = ((s.N + splits - 1) / splits + DM_ROWS - 1) / DM_ROWS * DM_ROWS;
    p.splits = (int)((s.N + p.n_per_split - 1) / p.n_per_split);
    p.w_bytes = ((size_t)s.O * s.I * RW * sizeof(double) + 255) & ~(size_t)255;
    p.slab_bytes = (size_t)s.O * s.I * RW * sizeof(double);
    return p;
}

template <typename F>
cudaError_t allow_smem(F* fn, size_t smem) {
    return smem > 48 * 1024 ? cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaSuccess;
}

cudaError_t pack_weights(const double* sw, const double* scaler, const double* bw, double* Wimg, const LayerShape& s,
                         cudaStream_t st) {
    const int64_t pairs = (int64_t)s.O * s.I;
    int blocks = (int)((pairs + 127) / 128);
    if (blocks > 148 * 8) blocks = 148 * 8;
    dm_pack_weights_kernel<<<blocks, 128, 0, st>>>(sw, scaler, bw, Wimg, s.O, s.I, s.R());
    return cudaGetLastError();
}

template <int K>
cudaError_t launch_forward(const double* x, const double* grid, const double* Wimg, double* y, const LayerShape& s,
                           const DmPlan& p, bool has_base, int* status, cudaStream_t st) {
    const int RW = s.R() + 1, ld = lead_dim(round_up(p.ci * RW, 4));
    const int64_t ntiles = (s.N + DM_ROWS - 1) / DM_ROWS;
    int bx = (int)(ntiles < 2 * 148 ? ntiles : 2 * 148);
    if (p.otiles > 1) bx = (int)(ntiles < 148 ? ntiles : 148);
    dim3 g(bx, p.otiles);
    cudaError_t e;
    if (p.to == 64) {
        const size_t smem = ((size_t)(DM_ROWS + 64) * ld + (size_t)p.ci * s.T() * (1 + s.K)) * sizeof(double);
        auto* fn = dm_forward_kernel<K, 2, 4, 4, 2>;
        if ((e = allow_smem(fn, smem)) != cudaSuccess) return e;
        fn<<<g, DM_THREADS, smem, st>>>(x, grid, Wimg, y, s.N, s.I, s.O, s.G, p.ci, has_base, status);
    } else {
        const size_t smem = ((size_t)(DM_ROWS + 8) * ld + (size_t)p.ci * s.T() * (1 + s.K)) * sizeof(double);
        auto* fn = dm_forward_kernel<K, 8, 1, 1, 1>;
        if ((e = allow_smem(fn, smem)) != cudaSuccess) return e;
        fn<<<g, DM_THREADS, smem, st>>>(x, grid, Wimg, y, s.N, s.I, s.O, s.G, p.ci, has_base, status);
    }
    return cudaGetLastError();
}

template <int K>
cudaError_t launch_bwd_param(const double* dY, const double* x, const double* grid, double* partial,
                             const LayerShape& s, const DmPlan& p, bool has_base, int* status, cudaStream_t st) {
    const int RW = s.R() + 1, lda = lead_dim(round_up(p.ci * RW, 8));
    dim3 g(p.groups, p.splits, p.otiles);
    if (g.y > 65535u || g.z > 65535u) return cudaErrorInvalidConfiguration;
    cudaError_t e;
    if (p.to == 64) {
        const size_t smem = ((size_t)DM_ROWS * (lda + lead_dim(64)) + (size_t)p.ci * s.T() * (1 + s.K)) * sizeof(double);
        auto* fn = dm_bwd_param_kernel<K, 2, 4, 2>;
        if ((e = allow_smem(fn, smem)) != cudaSuccess) return e;
        fn<<<g, DM_THREADS, smem, st>>>(dY, x, grid, partial, s.N, s.I, s.O, s.G, p.ci, has_base, p.n_per_split,
                                        status);
    } else {
        const size_t smem = ((size_t)DM_ROWS * (lda + lead_dim(8)) + (size_t)p.ci * s.T() * (1 + s.K)) * sizeof(double);
        auto* fn = dm_bwd_param_kernel<K, 8, 1, 1>;
        if ((e = allow_smem(fn, smem)) != cudaSuccess) return e;
        fn<<<g, DM_THREADS, smem, st>>>(dY, x, grid, partial, s.N, s.I, s.O, s.G, p.ci, has_base, p.n_per_split,
                                        status);
    }
    return cudaGetLastError();
}

template <int K>
cudaError_t launch_bwd_input(const double* dY, const double* x, const double* grid, const double* Wimg, double* gx,
                             const LayerShape& s, const DmPlan& p, bool has_base, int* status, cudaStream_t st) {
    const size_t smem = ((size_t)(DM_ROWS + DM_KO) * lead_dim(DM_CK_DX) + (size_t)DM_ROWS * lead_dim(DM_KO) +
                         (size_t)p.ci_dx * s.T() * (1 + s.K)) * sizeof(double);
    const int64_t ntiles = (s.N + DM_ROWS - 1) / DM_ROWS;
    // Every block walks all feature groups of its row tiles.  (One group per block with resident
    // weights -- gridDim.y = groups, which the kernel supports -- was measured slower, 1.44 against
    // 1.09 ms for 64 -> 64 at 131072 rows: the 40-byte pieces of x and gx rows that a group touches
    // are then fetched and written by different blocks at different times.)
    const int by = 1;
    int64_t bx = (2 * 148 + by - 1) / by;
    if (bx > ntiles) bx = ntiles;
    auto* fn = dm_bwd_input_kernel<K>;
    cudaError_t e = allow_smem(fn, smem);
    if (e != cudaSuccess) return e;
    fn<<<dim3((unsigned)bx, (unsigned)by), DM_THREADS, smem, st>>>(dY, x, grid, Wimg, gx, s.N, s.I, s.O, s.G, p.ci_dx, has_base, status);
    return cudaGetLastError();
}

#define KAN_DM_DISPATCH_K(Kval, ...)                               \
    switch (Kval) {                                                \
        case 1: { constexpr int KK = 1; __VA_ARGS__; break; }      \
        case 2: { constexpr int KK = 2; __VA_ARGS__; break; }      \
        default: { constexpr int KK = 3; __VA_ARGS__; break; }     \
    }

}  // namespace

bool dense64_supported(const LayerShape& s) {
    // (R + 1) <= 64 keeps at least one whole feature inside a chunk of the input-gradient kernel
    return s.K >= 1 && s.K <= 3 && s.N >= DM_MIN_ROWS && s.R() + 1 <= DM_CK_DX;
}

size_t dense64_workspace(bool forward, const LayerShape& s, bool need_x, bool need_param) {
    const DmPlan p = dm_plan(s);
    if (forward) return kWsHeader + p.w_bytes;
    return kWsHeader + (need_x ? p.w_bytes : 0) + (need_param ? (size_t)p.splits * p.slab_bytes : 0);
}

cudaError_t dense64_forward(const double* x, const double* grid, const double* bw, const double* sw,
                            const double* scaler, double* y, const LayerShape& s, void* ws, size_t ws_bytes,
                            cudaStream_t st) {
    const DmPlan p = dm_plan(s);
    if (!ws || ws_bytes < kWsHeader + p.w_bytes) return cudaErrorMemoryAllocation;
    int* status = reinterpret_cast<int*>(ws);
    double* Wimg = reinterpret_cast<double*>(reinterpret_cast<char*>(ws) + kWsHeader);
    cudaError_t e = pack_weights(sw, scaler, bw, Wimg, s, st);
    if (e != cudaSuccess) return e;
    KAN_DM_DISPATCH_K(s.K, (e = launch_forward<KK>(x, grid, Wimg, y, s, p, bw != nullptr, status, st)));
    return e;
}

cudaError_t dense64_backward(const double* dY, const double* x, const double* grid, const double* bw,
                             const double* sw, const double* scaler, double* gx, double* gbw, double* gsw,
                             double* gscaler, const LayerShape& s, void* ws, size_t ws_bytes, cudaStream_t st) {
    const DmPlan p = dm_plan(s);
    const bool need_param = gbw || gsw || gscaler;
    const size_t need = (gx ? p.w_bytes : 0) + (need_param ? (size_t)p.splits * p.slab_bytes : 0);
    if (!ws || ws_bytes < kWsHeader + need) return cudaErrorMemoryAllocation;
    int* status = reinterpret_cast<int*>(ws);
    char* base = reinterpret_cast<char*>(ws) + kWsHeader;
    cudaError_t e = cudaSuccess;
    if (need_param) {
        double* partial = reinterpret_cast<double*>(base + (gx ? p.w_bytes : 0));
        KAN_DM_DISPATCH_K(s.K, (e = launch_bwd_param<KK>(dY, x, grid, partial, s, p, bw != nullptr, status, st)));
        if (e != cudaSuccess) return e;
        const int RW = s.R() + 1;
        e = finalize_param_grads<double>(partial, p.splits, (int64_t)s.O * s.I * RW, (int64_t)s.I * RW, RW, s.R(),
                                         RW, sw, scaler, gsw, gscaler, bw ? gbw : nullptr, s.O, s.I, s.R(), st);
        if (e != cudaSuccess) return e;
    }
    if (gx) {
        double* Wimg = reinterpret_cast<double*>(base);
        e = pack_weights(sw, scaler, bw, Wimg, s, st);
        if (e != cudaSuccess) return e;
        KAN_DM_DISPATCH_K(s.K, (e = launch_bwd_input<KK>(dY, x, grid, Wimg, gx, s, p, bw != nullptr, status, st)));
    }
    return e;
}

}  // namespace kanb200
