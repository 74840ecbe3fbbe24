// Tensor-core (tcgen05 / TMEM) kernels of the KANLinear path for fp32 tensors.
//
// The spline contraction  y[n,o] = sum_{i,r} B_r(x[n,i]) W_eff[o,i,r] + sum_i silu(x[n,i]) bw[o,i]
// is a dense GEMM whose left operand is never stored: its tiles are evaluated
// from x in registers and written straight into the shared-memory operand
// layout the MMA unit reads.  fp32 accuracy is kept on 16-bit tensor-core
// inputs by splitting every operand value v into hi = bf16(v) and
// lo = bf16(v - hi) and issuing three MMAs per step (hi*hi + lo*hi + hi*lo).
//
// Column space ("c") of the generated operand, shared by all kernels:
//   spline part : c = i * 8 + r            (R <= 8, slots r >= R are zero)
//   base part   : c = CS + i               (CS = 8 * I rounded up to 256)
//
// Kernels
//   pack_weights_kernel    W_eff / base_weight -> bf16 hi/lo tile images
//   pack_grad_out_kernel   dY                  -> bf16 hi/lo tile images
//   tc_forward_kernel      y   = A(x) W^T           M = samples,  K = c
//   tc_bwd_param_kernel    D   = dY^T A(x)          M = outputs,  K = samples
// All are persistent, warp-specialised (bulk-copy thread, MMA thread, operand
// producer warps, epilogue warps) and every wait is bounded.
#include "kan_device.cuh"
#include "kan_internal.h"
#include "kan_tc_ptx.cuh"

namespace kanb200 {

namespace {

using namespace ptx;

constexpr int kStatusTimeout = 1;
constexpr int kStatusBadSmem = 2;

constexpr int BLOCK_M = 128;       // accumulator rows (TMEM lanes)
constexpr int BLOCK_N = 256;       // accumulator columns per MMA
constexpr int BLOCK_K = 64;        // bf16 elements per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int RP = 8;              // spline slots per feature in the column space

constexpr uint32_t TILE_A_BYTES = BLOCK_M * BLOCK_K * 2;   // 16 KB: 128 x 64 bf16
constexpr uint32_t TILE_B_BYTES = BLOCK_N * BLOCK_K * 2;   // 32 KB: 256 x 64 bf16

// ---------------------------------------------------------------------------
// Local basis with approximate reciprocals (2 ulp) for the operand producers.
// ---------------------------------------------------------------------------
template <int K>
__device__ __forceinline__ void local_basis_fast(const float* __restrict__ t, int nk, int m, float x,
                                                 float (&val)[K + 1]) {
    float tk[2 * K];
#pragma unroll
    for (int q = 0; q < 2 * K; ++q) {
        int idx = m - K + 1 + q;
        idx = idx < 0 ? 0 : (idx > nk - 1 ? nk - 1 : idx);
        tk[q] = t[idx];
    }
    float nd[K + 1];
    nd[0] = 1.0f;
#pragma unroll
    for (int j = 1; j <= K; ++j) nd[j] = 0.0f;
#pragma unroll
    for (int d = 1; d <= K; ++d) {
        float carry = 0.0f;
#pragma unroll
        for (int j = 0; j < d; ++j) {
            const float hi_k = tk[K + j], lo_k = tk[K - d + j];
            const float den = hi_k - lo_k;
            const float w = (den != 0.0f) ? __fdividef(nd[j], den) : 0.0f;
            nd[j] = fmaf(hi_k - x, w, carry);
            carry = (x - lo_k) * w;
        }
        nd[d] = carry;
    }
#pragma unroll
    for (int j = 0; j <= K; ++j) val[j] = nd[j];
}

// Span of x among nk <= 12 sorted knots: compare-and-count (knot reads are
// warp-uniform or conflict-free shared-memory reads).
__device__ __forceinline__ int span_by_count(const float* __restrict__ t, int nk, float x) {
    if (!(x >= t[0]) || !(x <= t[nk - 1])) return -1;
    int c = 0;
#pragma unroll
    for (int q = 1; q <= 10; ++q)
        if (q < nk - 1) c += (x >= t[q]) ? 1 : 0;
    return c;
}

__device__ __forceinline__ float silu_fast(float x) {
    return __fdividef(x, 1.0f + __expf(-x));
}

// Evaluates the basis of one input and returns the 8 column slots of its
// feature as two 128-bit rows (hi and lo bf16 parts).  SPLIT = false leaves lo
// untouched.
template <int K, bool SPLIT>
__device__ __forceinline__ void eval_feature_row(const float* __restrict__ t, int nk, int R, float xv,
                                                 uint4& hi, uint4& lo) {
    const int m = span_by_count(t, nk, xv);
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int s = 0;
    if (m >= 0) {
        float w[K + 1];
        local_basis_fast<K>(t, nk, m, xv, w);
        s = m - K;
#pragma unroll
        for (int j = 0; j <= K; ++j) {
            const int r = s + j;
            v[j] = (r >= 0 && r < R) ? w[j] : 0.0f;
        }
    }
    uint32_t h01, h23, l01 = 0, l23 = 0;
    if (SPLIT) {
        split2(v[0], v[1], h01, l01);
        split2(v[2], v[3], h23, l23);
    } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
        h01 = *reinterpret_cast<const uint32_t*>(&a);
        h23 = *reinterpret_cast<const uint32_t*>(&b);
    }
    // Place the 4 half-words at half-word offset s (in [-3, 7]) of a 128-bit row.
    auto place = [&](uint32_t w01, uint32_t w23) -> uint4 {
        const uint64_t p = (uint64_t)w01 | ((uint64_t)w23 << 32);
        uint64_t lo64, hi64;
        if (s >= 0) {
            const int nb = 16 * s;
            lo64 = (nb < 64) ? (p << nb) : 0ull;
            hi64 = (nb == 0) ? 0ull : ((nb < 64) ? (p >> (64 - nb)) : (p << (nb - 64)));
        } else {
            lo64 = p >> (-16 * s);
            hi64 = 0ull;
        }
        return make_uint4((uint32_t)lo64, (uint32_t)(lo64 >> 32), (uint32_t)hi64, (uint32_t)(hi64 >> 32));
    };
    hi = place(h01, h23);
    if (SPLIT) lo = place(l01, l23);
}

// 8 consecutive silu values -> one 16-byte chunk (hi) and one (lo).
template <bool SPLIT>
__device__ __forceinline__ void silu_chunk(const float (&xv)[8], uint4& hi, uint4& lo) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = silu_fast(xv[e]);
    uint32_t h[4], l[4] = {0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (SPLIT) {
            split2(s[2 * e], s[2 * e + 1], h[e], l[e]);
        } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(s[2 * e], s[2 * e + 1]);
            h[e] = *reinterpret_cast<const uint32_t*>(&a);
        }
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Loads 8 consecutive floats x[row, f0 .. f0+7] (zero beyond I or when !row_ok).
__device__ __forceinline__ void load_x8(const float* __restrict__ x, int64_t row, bool row_ok, int I, int f0,
                                        bool vec_ok, float (&out)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = 0.0f;
    if (!row_ok || f0 >= I) return;
    const float* p = x + (size_t)row * I + f0;
    if (vec_ok && f0 + 8 <= I) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p));
        const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (f0 + e < I) out[e] = __ldg(p + e);
    }
}

// ---------------------------------------------------------------------------
// Weight images.  For every (o-tile of 256, k-block of 64 columns) the image
// holds two 32-KB tiles (hi, lo) that are byte-for-byte the shared-memory
// contents the MMA unit expects: 256 rows (outputs) x 128 B (64 columns),
// 128-byte swizzle.  One bulk copy brings a tile in.
// ---------------------------------------------------------------------------
struct ColumnSpace {
    int kb_spline;     // k-blocks (64 columns = 8 features) of the spline part
    int kb_base;       // k-blocks (64 features) of the base part, 0 without base
    int kb_total() const { return kb_spline + kb_base; }
};

inline ColumnSpace column_space(int I, bool has_base) {
    ColumnSpace c;
    c.kb_spline = (I + 7) / 8;
    c.kb_base = has_base ? (I + 63) / 64 : 0;
    return c;
}

__global__ void pack_weights_kernel(const float* __restrict__ sw, const float* __restrict__ scaler,
                                    const float* __restrict__ bw, uint8_t* __restrict__ img,
                                    int O, int I, int R, int kb_spline, int kb_total, int n_otiles) {
    // one thread per 16-byte chunk: (o_row in tile, chunk 0..7) of one (o-tile, k-block)
    const int64_t chunks = (int64_t)n_otiles * kb_total * BLOCK_N * 8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < chunks;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int cc = (int)(idx & 7);
        int64_t rest = idx >> 3;
        const int kb = (int)(rest % kb_total);
        rest /= kb_total;
        const int rr = (int)(rest % BLOCK_N);
        const int ot = (int)(rest / BLOCK_N);
        const int o = ot * BLOCK_N + rr;
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = 0.0f;
        if (o < O) {
            if (kb < kb_spline) {
                const int f = kb * 8 + cc;
                if (f < I) {
                    const size_t oi = (size_t)o * I + f;
                    const float sc = scaler ? scaler[oi] : 1.0f;
                    for (int e = 0; e < 8; ++e)
                        if (e < R) {
                            const float v = sw[oi * R + e];
                            w[e] = scaler ? v * sc : v;
                        }
                }
            } else {
                const int f0 = (kb - kb_spline) * 64 + cc * 8;
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (f0 + e < I) w[e] = bw[(size_t)o * I + f0 + e];
            }
        }
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split2(w[2 * e], w[2 * e + 1], h[e], l[e]);
        uint8_t* tile = img + ((size_t)ot * kb_total + kb) * (2 * (size_t)TILE_B_BYTES);
        const uint32_t off = sw128_chunk_offset((uint32_t)rr, (uint32_t)cc);
        *reinterpret_cast<uint4*>(tile + off) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(tile + TILE_B_BYTES + off) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

// dY images for the parameter-gradient kernel.  For every (block of 64
// samples, group of 128 outputs) two 16-KB tiles (hi, lo), MN-major: rows are
// samples, 128 B = 64 consecutive outputs, 128-byte swizzle, laid out
// [output group of 64][sample group of 8][8 rows][128 B].
__global__ void pack_grad_out_kernel(const float* __restrict__ dY, uint8_t* __restrict__ img,
                                     int64_t N, int O, int64_t n_blocks, int n_ohalves) {
    const int64_t chunks = n_blocks * n_ohalves * 64 * 16;   // 64 samples x 16 chunks of 8 outputs
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < chunks;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int oc = (int)(idx & 15);            // chunk of 8 outputs within the 128
        int64_t rest = idx >> 4;
        const int oh = (int)(rest % n_ohalves);
        rest /= n_ohalves;
        const int nn = (int)(rest & 63);
        const int64_t nb = rest >> 6;
        const int64_t n = nb * 64 + nn;
        const int o0 = oh * 128 + oc * 8;
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = 0.0f;
        if (n < N) {
            const float* p = dY + (size_t)n * O + o0;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (o0 + e < O) w[e] = p[e];
        }
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split2(w[2 * e], w[2 * e + 1], h[e], l[e]);
        uint8_t* tile = img + ((size_t)nb * n_ohalves + oh) * (2 * (size_t)TILE_A_BYTES);
        const int og = oc >> 3, ch = oc & 7, kg = nn >> 3, kk = nn & 7;
        const uint32_t off = (uint32_t)(og * 8 + kg) * 1024u + (uint32_t)kk * 128u + (uint32_t)((ch ^ kk) << 4);
        *reinterpret_cast<uint4*>(tile + off) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(tile + TILE_A_BYTES + off) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

// ---------------------------------------------------------------------------
// Forward kernel
// ---------------------------------------------------------------------------
constexpr int FWD_EPI_WARPS = 4, FWD_PROD_WARPS = 8;
constexpr int FWD_THREADS = (FWD_EPI_WARPS + FWD_PROD_WARPS + 2) * 32;   // 448
constexpr int FWD_A_STAGES = 2, FWD_B_SLOTS = 5;
constexpr uint32_t FWD_A_STAGE_BYTES = 2 * TILE_A_BYTES;                  // hi + lo
constexpr uint32_t FWD_SMEM_A = 0;
constexpr uint32_t FWD_SMEM_B = FWD_SMEM_A + FWD_A_STAGES * FWD_A_STAGE_BYTES;
constexpr uint32_t FWD_SMEM_CTRL = FWD_SMEM_B + FWD_B_SLOTS * TILE_B_BYTES;
constexpr uint32_t FWD_KNOT_FLOATS = 4 * 12;                              // per producer warp
constexpr uint32_t FWD_CTRL_BYTES = 256 + FWD_PROD_WARPS * FWD_KNOT_FLOATS * 4;
constexpr uint32_t FWD_SMEM_BYTES = FWD_SMEM_CTRL + FWD_CTRL_BYTES;
static_assert(FWD_SMEM_BYTES <= 232448, "forward kernel shared memory exceeds 227 KB");

struct FwdCtrl {
    uint64_t fullA[FWD_A_STAGES], emptyA[FWD_A_STAGES];
    uint64_t fullB[FWD_B_SLOTS], emptyB[FWD_B_SLOTS];
    uint64_t accFull[2], accEmpty[2];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(FwdCtrl) <= 256, "control block too large");

template <int K, int NTERMS>
__global__ void __launch_bounds__(FWD_THREADS, 1)
tc_forward_kernel(const float* __restrict__ x, const float* __restrict__ grid, const uint8_t* __restrict__ wimg,
                  float* __restrict__ y, int* __restrict__ status,
                  int64_t N, int I, int O, int G, int kb_spline, int kb_total,
                  int n_otiles, int64_t n_tiles, int vec_ok) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    FwdCtrl* ctrl = reinterpret_cast<FwdCtrl*>(smem + FWD_SMEM_CTRL);
    float* knot_stage = reinterpret_cast<float*>(smem + FWD_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = G + K, nk = G + 2 * K + 1;

    if ((sbase & 1023u) != 0) {                 // swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicExch(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < FWD_A_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullA[s]), FWD_PROD_WARPS * 32);
            mbar_init(smem_u32(&ctrl->emptyA[s]), 1);
        }
        for (int s = 0; s < FWD_B_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullB[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyB[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctrl->accFull[s]), 1);
            mbar_init(smem_u32(&ctrl->accEmpty[s]), FWD_EPI_WARPS * 32);
        }
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    constexpr int MMA_WARP = FWD_EPI_WARPS + FWD_PROD_WARPS, TMA_WARP = MMA_WARP + 1;
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp < FWD_EPI_WARPS) {
        // ===== epilogue: TMEM -> registers -> y =====
        const int row = warp * 32 + lane;
        uint32_t tcount = 0;
        for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tcount) {
            const int64_t mt = tile / n_otiles;
            const int ot = (int)(tile - mt * n_otiles);
            const uint32_t buf = tcount & 1u;
            if (!mbar_wait(smem_u32(&ctrl->accFull[buf]), (tcount >> 1) & 1u, abort_flag)) break;
            tc_fence_after_sync();
            const int64_t n = mt * BLOCK_M + row;
            float* yrow = y + (size_t)n * O + (size_t)ot * BLOCK_N;
            const int ocount = O - ot * BLOCK_N;           // valid columns in this tile (may exceed 256)
            const bool vec_store = ((O & 3) == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
#pragma unroll 1
            for (int c = 0; c < BLOCK_N / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BLOCK_N + c * 32, r);
                tmem_ld_wait();
                if (n < N) {
                    const int c0 = c * 32;
                    if (vec_store && c0 + 32 <= ocount) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<float4*>(yrow + c0 + 4 * q) =
                                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                            __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                    } else {
#pragma unroll
                        for (int q = 0; q < 32; ++q)
                            if (c0 + q < ocount) yrow[c0 + q] = __uint_as_float(r[q]);
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->accEmpty[buf]));
        }
    } else if (warp < FWD_EPI_WARPS + FWD_PROD_WARPS) {
        // ===== operand producers: x -> basis / silu -> swizzled bf16 A tile =====
        const int pw = warp - FWD_EPI_WARPS;
        const int row = (pw & 3) * 32 + lane;
        const int half = pw >> 2;                         // which half of the k-block's chunks
        float* kn = knot_stage + pw * FWD_KNOT_FLOATS;    // this warp's knots of 4 features
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int64_t mt = tile / n_otiles;
            const int64_t n = mt * BLOCK_M + row;
            const bool row_ok = n < N;
            for (int kb = 0; kb < kb_total; ++kb, ++it) {
                const uint32_t stage = it % FWD_A_STAGES;
                const uint32_t a_hi = sbase + FWD_SMEM_A + stage * FWD_A_STAGE_BYTES;
                const uint32_t a_lo = a_hi + TILE_A_BYTES;
                if (kb < kb_spline) {
                    const int f0 = kb * 8 + half * 4;
                    float xv[4] = {0.f, 0.f, 0.f, 0.f};
                    if (row_ok && f0 < I) {
                        const float* p = x + (size_t)n * I + f0;
                        if (vec_ok && f0 + 4 <= I) {
                            const float4 a = __ldg(reinterpret_cast<const float4*>(p));
                            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (f0 + e < I) xv[e] = __ldg(p + e);
                        }
                    }
                    __syncwarp();
                    for (int e = lane; e < 4 * nk; e += 32) {
                        const int f = f0 + e / nk;
                        kn[e] = (f < I) ? __ldg(grid + (size_t)f0 * nk + e) : 0.0f;
                    }
                    __syncwarp();
                    if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / FWD_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        uint4 hi, lo;
                        if (row_ok && f0 + e < I) {
                            eval_feature_row<K, SPLIT>(kn + e * nk, nk, R, xv[e], hi, lo);
                        } else {
                            hi = make_uint4(0, 0, 0, 0);
                            lo = hi;
                        }
                        const uint32_t off = sw128_chunk_offset((uint32_t)row, (uint32_t)(half * 4 + e));
                        st_shared_v4(a_hi + off, hi);
                        if (SPLIT) st_shared_v4(a_lo + off, lo);
                    }
                } else {
                    const int f0 = (kb - kb_spline) * 64 + half * 32;
                    float xv[4][8];
#pragma unroll
                    for (int c = 0; c < 4; ++c) load_x8(x, n, row_ok, I, f0 + c * 8, vec_ok != 0, xv[c]);
                    if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / FWD_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 hi, lo;
                        silu_chunk<SPLIT>(xv[c], hi, lo);
                        const uint32_t off = sw128_chunk_offset((uint32_t)row, (uint32_t)(half * 4 + c));
                        st_shared_v4(a_hi + off, hi);
                        if (SPLIT) st_shared_v4(a_lo + off, lo);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullA[stage]));
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // ===== MMA issue =====
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, false, false);
            constexpr uint64_t dbase = make_sdesc_sw128(16, 1024);
            uint32_t it = 0, bslot = 0, tcount = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tcount) {
                const uint32_t buf = tcount & 1u;
                if (!mbar_wait(smem_u32(&ctrl->accEmpty[buf]), ((tcount >> 1) & 1u) ^ 1u, abort_flag)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
                for (int kb = 0; kb < kb_total; ++kb, ++it) {
                    const uint32_t stage = it % FWD_A_STAGES;
                    const uint32_t a_hi = sbase + FWD_SMEM_A + stage * FWD_A_STAGE_BYTES;
                    const uint32_t a_lo = a_hi + TILE_A_BYTES;
                    const uint32_t slot_h = bslot % FWD_B_SLOTS;
                    const uint32_t par_h = (bslot / FWD_B_SLOTS) & 1u;
                    if (!mbar_wait(smem_u32(&ctrl->fullA[stage]), (it / FWD_A_STAGES) & 1u, abort_flag) ||
                        !mbar_wait(smem_u32(&ctrl->fullB[slot_h]), par_h, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t b_hi = sbase + FWD_SMEM_B + slot_h * TILE_B_BYTES;
#pragma unroll
                    for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                        mma_f16_ss(d_tmem, sdesc_at(dbase, a_hi + ks * 32), sdesc_at(dbase, b_hi + ks * 32), idesc,
                                   (kb > 0 || ks > 0) ? 1u : 0u);
                    if (SPLIT) {
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, a_lo + ks * 32), sdesc_at(dbase, b_hi + ks * 32),
                                       idesc, 1u);
                    }
                    mma_commit(smem_u32(&ctrl->emptyB[slot_h]));
                    ++bslot;
                    if (SPLIT) {
                        const uint32_t slot_l = bslot % FWD_B_SLOTS;
                        const uint32_t par_l = (bslot / FWD_B_SLOTS) & 1u;
                        if (!mbar_wait(smem_u32(&ctrl->fullB[slot_l]), par_l, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t b_lo = sbase + FWD_SMEM_B + slot_l * TILE_B_BYTES;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, a_hi + ks * 32), sdesc_at(dbase, b_lo + ks * 32),
                                       idesc, 1u);
                        mma_commit(smem_u32(&ctrl->emptyB[slot_l]));
                        ++bslot;
                    }
                    mma_commit(smem_u32(&ctrl->emptyA[stage]));
                }
                if (ok) mma_commit(smem_u32(&ctrl->accFull[buf]));
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk-copy producer for weight tiles =====
            uint32_t bslot = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int64_t mt = tile / n_otiles;
                const int ot = (int)(tile - mt * n_otiles);
                for (int kb = 0; kb < kb_total && ok; ++kb) {
                    const uint8_t* src = wimg + ((size_t)ot * kb_total + kb) * (2 * (size_t)TILE_B_BYTES);
                    for (int term = 0; term < (SPLIT ? 2 : 1); ++term, ++bslot) {
                        const uint32_t slot = bslot % FWD_B_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->emptyB[slot]), ((bslot / FWD_B_SLOTS) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = smem_u32(&ctrl->fullB[slot]);
                        mbar_arrive_expect_tx(bar, TILE_B_BYTES);
                        bulk_g2s(sbase + FWD_SMEM_B + slot * TILE_B_BYTES, src + (size_t)term * TILE_B_BYTES,
                                 TILE_B_BYTES, bar);
                    }
                }
            }
        }
    }

    // ===== teardown =====
    if (*abort_flag) {
        if (lane == 0) atomicExch(status, kStatusTimeout);
        __nanosleep(100000);                   // let copies / MMAs in flight land
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == MMA_WARP) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------
// Parameter-gradient kernel:  D[o, c] = sum_n dY[n, o] A[n, c]
// ---------------------------------------------------------------------------
// Work item = (output tile of 256, column tile of 256, sample split).  The
// accumulator is two 128-row halves (all 512 TMEM columns).  Both operands are
// MN-major: dY tiles come in as pre-swizzled images by bulk copy, the basis /
// silu operand is generated by the producer warps.
constexpr int BWD_EPI_WARPS = 4, BWD_PROD_WARPS = 8;
constexpr int BWD_THREADS = (BWD_EPI_WARPS + BWD_PROD_WARPS + 2) * 32;
constexpr int BWD_G_STAGES = 2, BWD_D_SLOTS = 3;
constexpr uint32_t BWD_G_STAGE_BYTES = 2 * TILE_B_BYTES;                 // hi + lo, 256 c x 64 n
constexpr uint32_t BWD_D_SLOT_BYTES = 2 * TILE_A_BYTES;                  // hi + lo, 128 o x 64 n
constexpr uint32_t BWD_SMEM_G = 0;
constexpr uint32_t BWD_SMEM_D = BWD_SMEM_G + BWD_G_STAGES * BWD_G_STAGE_BYTES;
constexpr uint32_t BWD_SMEM_CTRL = BWD_SMEM_D + BWD_D_SLOTS * BWD_D_SLOT_BYTES;
constexpr uint32_t BWD_KNOT_STRIDE = 13;
constexpr uint32_t BWD_CTRL_BYTES = 256 + 32 * BWD_KNOT_STRIDE * 4;
constexpr uint32_t BWD_SMEM_BYTES = BWD_SMEM_CTRL + BWD_CTRL_BYTES;
static_assert(BWD_SMEM_BYTES <= 232448, "backward kernel shared memory exceeds 227 KB");

struct BwdCtrl {
    uint64_t fullG[BWD_G_STAGES], emptyG[BWD_G_STAGES];
    uint64_t fullD[BWD_D_SLOTS], emptyD[BWD_D_SLOTS];
    uint64_t accFull, accEmpty;
    uint64_t prodBar;      // producer-warp rendezvous around the per-item knot reload
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(BwdCtrl) <= 256, "control block too large");

struct BwdPlan {
    int n_otiles;          // tiles of 256 outputs
    int ct_spline;         // column tiles of 32 features
    int ct_base;           // column tiles of 256 base features
    int splits;
    int64_t kb_total;      // 64-sample blocks
    int64_t kb_per_split;
    __host__ __device__ int n_ctiles() const { return ct_spline + ct_base; }
    __host__ __device__ int64_t n_items() const { return (int64_t)n_otiles * n_ctiles() * splits; }
    __host__ __device__ int64_t ld_partial() const { return (int64_t)n_ctiles() * BLOCK_N; }
};

template <int K, int NTERMS>
__global__ void __launch_bounds__(BWD_THREADS, 1)
tc_bwd_param_kernel(const float* __restrict__ x, const float* __restrict__ grid, const uint8_t* __restrict__ dyimg,
                    float* __restrict__ partial, int* __restrict__ status,
                    int64_t N, int I, int O, int G, BwdPlan plan, int vec_ok) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    BwdCtrl* ctrl = reinterpret_cast<BwdCtrl*>(smem + BWD_SMEM_CTRL);
    float* knots = reinterpret_cast<float*>(smem + BWD_SMEM_CTRL + 256);    // [32][13]
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = G + K, nk = G + 2 * K + 1;
    const int n_ohalves = plan.n_otiles * 2;
    const int n_ctiles = plan.n_ctiles();
    const int64_t n_items = plan.n_items();

    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < BWD_G_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullG[s]), BWD_PROD_WARPS * 32);
            mbar_init(smem_u32(&ctrl->emptyG[s]), 1);
        }
        for (int s = 0; s < BWD_D_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullD[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyD[s]), 1);
        }
        mbar_init(smem_u32(&ctrl->accFull), 1);
        mbar_init(smem_u32(&ctrl->accEmpty), BWD_EPI_WARPS * 32);
        mbar_init(smem_u32(&ctrl->prodBar), BWD_PROD_WARPS * 32);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    constexpr int MMA_WARP = BWD_EPI_WARPS + BWD_PROD_WARPS, TMA_WARP = MMA_WARP + 1;
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    // item -> (split, o-tile, c-tile); consecutive items share the o-tile.
    auto decode = [&](int64_t item, int& sp, int& ot, int& ct) {
        ct = (int)(item % n_ctiles);
        const int64_t rest = item / n_ctiles;
        ot = (int)(rest % plan.n_otiles);
        sp = (int)(rest / plan.n_otiles);
    };

    if (warp < BWD_EPI_WARPS) {
        // ===== epilogue: both accumulator halves -> partial slab =====
        uint32_t icount = 0;
        for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x, ++icount) {
            int sp, ot, ct;
            decode(item, sp, ot, ct);
            if (!mbar_wait(smem_u32(&ctrl->accFull), icount & 1u, abort_flag)) break;
            tc_fence_after_sync();
            float* slab = partial + (size_t)sp * ((size_t)O * plan.ld_partial());
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const int o = ot * BLOCK_N + h * BLOCK_M + warp * 32 + lane;
                float* prow = slab + (size_t)o * plan.ld_partial() + (size_t)ct * BLOCK_N;
#pragma unroll 1
                for (int c = 0; c < BLOCK_N / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + h * BLOCK_N + c * 32, r);
                    tmem_ld_wait();
                    if (o < O) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<float4*>(prow + c * 32 + 4 * q) =
                                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                            __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->accEmpty));
        }
    } else if (warp < BWD_EPI_WARPS + BWD_PROD_WARPS) {
        // ===== operand producers: 64 samples x 256 columns, MN-major =====
        const int pw = warp - BWD_EPI_WARPS;
        const int ptid = pw * 32 + lane;
        uint32_t it = 0, sync_phase = 0;
        bool ok = true;
        // Bounded rendezvous of the producer warps (an mbarrier, not bar.sync,
        // so that a role that gave up cannot leave the others waiting forever).
        auto producer_sync = [&]() -> bool {
            const uint32_t bar = smem_u32(&ctrl->prodBar);
            mbar_arrive(bar);
            const bool r = mbar_wait(bar, sync_phase & 1u, abort_flag);
            ++sync_phase;
            return r;
        };
        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int sp, ot, ct;
            decode(item, sp, ot, ct);
            const bool spline = ct < plan.ct_spline;
            const int f_tile0 = spline ? ct * 32 : (ct - plan.ct_spline) * 256;
            if (spline) {
                if (!producer_sync()) break;       // previous item's knot reads are done
                for (int e = ptid; e < 32 * nk; e += BWD_PROD_WARPS * 32) {
                    const int fl = e / nk, q = e - fl * nk;
                    const int f = f_tile0 + fl;
                    knots[fl * BWD_KNOT_STRIDE + q] = (f < I) ? __ldg(grid + (size_t)f * nk + q) : 0.0f;
                }
                if (!producer_sync()) break;
            }
            const int64_t kb0 = (int64_t)sp * plan.kb_per_split;
            int64_t kb1 = kb0 + plan.kb_per_split;
            if (kb1 > plan.kb_total) kb1 = plan.kb_total;
            for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t stage = it % BWD_G_STAGES;
                const uint32_t g_hi = sbase + BWD_SMEM_G + stage * BWD_G_STAGE_BYTES;
                const uint32_t g_lo = g_hi + TILE_B_BYTES;
                // this warp's 8 samples of the block: rows pw*8 .. pw*8+7 = one group of 8 K rows
                const int64_t nrow0 = kb * BLOCK_K + pw * 8;
                if (spline) {
                    const int f = f_tile0 + lane;
                    float xv[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        xv[q] = (nrow0 + q < N && f < I) ? __ldg(x + (size_t)(nrow0 + q) * I + f) : 0.0f;
                    if (!mbar_wait(smem_u32(&ctrl->emptyG[stage]), ((it / BWD_G_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t atom = (uint32_t)((lane >> 3) * 8 + pw) * 1024u;   // [col group][sample group]
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        uint4 hi, lo;
                        if (nrow0 + q < N && f < I) {
                            eval_feature_row<K, SPLIT>(knots + lane * BWD_KNOT_STRIDE, nk, R, xv[q], hi, lo);
                        } else {
                            hi = make_uint4(0, 0, 0, 0);
                            lo = hi;
                        }
                        const uint32_t off = atom + (uint32_t)q * 128u + (uint32_t)(((lane & 7) ^ q) << 4);
                        st_shared_v4(g_hi + off, hi);
                        if (SPLIT) st_shared_v4(g_lo + off, lo);
                    }
                } else {
                    // lane = chunk of 8 base features; columns c = 8*lane .. 8*lane+7
                    const int f0 = f_tile0 + lane * 8;
                    if (!mbar_wait(smem_u32(&ctrl->emptyG[stage]), ((it / BWD_G_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t atom = (uint32_t)((lane >> 3) * 8 + pw) * 1024u;
#pragma unroll 2
                    for (int q = 0; q < 8; ++q) {
                        float xv[8];
                        load_x8(x, nrow0 + q, nrow0 + q < N, I, f0, vec_ok != 0, xv);
                        uint4 hi, lo;
                        silu_chunk<SPLIT>(xv, hi, lo);
                        if (!(nrow0 + q < N)) {
                            hi = make_uint4(0, 0, 0, 0);
                            lo = hi;
                        }
                        const uint32_t off = atom + (uint32_t)q * 128u + (uint32_t)(((lane & 7) ^ q) << 4);
                        st_shared_v4(g_hi + off, hi);
                        if (SPLIT) st_shared_v4(g_lo + off, lo);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullG[stage]));
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, true, true);
            constexpr uint64_t dbase = make_sdesc_sw128(8192, 1024);
            uint32_t it = 0, dslot = 0, icount = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++icount) {
                int sp, ot, ct;
                decode(item, sp, ot, ct);
                if (!mbar_wait(smem_u32(&ctrl->accEmpty), (icount & 1u) ^ 1u, abort_flag)) break;
                tc_fence_after_sync();
                const int64_t kb0 = (int64_t)sp * plan.kb_per_split;
                int64_t kb1 = kb0 + plan.kb_per_split;
                if (kb1 > plan.kb_total) kb1 = plan.kb_total;
                for (int64_t kb = kb0; kb < kb1 && ok; ++kb, ++it) {
                    const uint32_t stage = it % BWD_G_STAGES;
                    const uint32_t g_hi = sbase + BWD_SMEM_G + stage * BWD_G_STAGE_BYTES;
                    const uint32_t g_lo = g_hi + TILE_B_BYTES;
                    if (!mbar_wait(smem_u32(&ctrl->fullG[stage]), (it / BWD_G_STAGES) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    for (int h = 0; h < 2; ++h, ++dslot) {
                        const uint32_t slot = dslot % BWD_D_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->fullD[slot]), (dslot / BWD_D_SLOTS) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t d_hi = sbase + BWD_SMEM_D + slot * BWD_D_SLOT_BYTES;
                        const uint32_t d_lo = d_hi + TILE_A_BYTES;
                        const uint32_t d_tmem = tmem_base + h * BLOCK_N;
                        const uint32_t first = (kb > kb0) ? 1u : 0u;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, d_hi + ks * 2048), sdesc_at(dbase, g_hi + ks * 2048),
                                       idesc, (first || ks > 0) ? 1u : 0u);
                        if (SPLIT) {
#pragma unroll
                            for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                                mma_f16_ss(d_tmem, sdesc_at(dbase, d_lo + ks * 2048),
                                           sdesc_at(dbase, g_hi + ks * 2048), idesc, 1u);
#pragma unroll
                            for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                                mma_f16_ss(d_tmem, sdesc_at(dbase, d_hi + ks * 2048),
                                           sdesc_at(dbase, g_lo + ks * 2048), idesc, 1u);
                        }
                        mma_commit(smem_u32(&ctrl->emptyD[slot]));
                    }
                    if (ok) mma_commit(smem_u32(&ctrl->emptyG[stage]));
                }
                if (ok) mma_commit(smem_u32(&ctrl->accFull));
            }
        }
    } else {
        if (lane == 0) {
            uint32_t dslot = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int sp, ot, ct;
                decode(item, sp, ot, ct);
                const int64_t kb0 = (int64_t)sp * plan.kb_per_split;
                int64_t kb1 = kb0 + plan.kb_per_split;
                if (kb1 > plan.kb_total) kb1 = plan.kb_total;
                for (int64_t kb = kb0; kb < kb1 && ok; ++kb) {
                    for (int h = 0; h < 2; ++h, ++dslot) {
                        const uint32_t slot = dslot % BWD_D_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->emptyD[slot]), ((dslot / BWD_D_SLOTS) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        const uint8_t* src = dyimg + ((size_t)kb * n_ohalves + (size_t)(ot * 2 + h)) * BWD_D_SLOT_BYTES;
                        const uint32_t bytes = SPLIT ? BWD_D_SLOT_BYTES : TILE_A_BYTES;
                        const uint32_t bar = smem_u32(&ctrl->fullD[slot]);
                        mbar_arrive_expect_tx(bar, bytes);
                        bulk_g2s(sbase + BWD_SMEM_D + slot * BWD_D_SLOT_BYTES, src, bytes, bar);
                    }
                }
            }
        }
    }

    if (*abort_flag) {
        if (lane == 0) atomicExch(status, kStatusTimeout);
        __nanosleep(100000);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == MMA_WARP) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

inline int sm_count() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            cached = n;
        else
            cached = 148;
    }
    return cached;
}

inline BwdPlan plan_bwd(const LayerShape& s, bool has_base) {
    BwdPlan p;
    p.n_otiles = (s.O + BLOCK_N - 1) / BLOCK_N;
    p.ct_spline = (s.I + 31) / 32;
    p.ct_base = has_base ? (s.I + 255) / 256 : 0;
    p.kb_total = (s.N + BLOCK_K - 1) / BLOCK_K;
    const int64_t tiles = (int64_t)p.n_otiles * p.n_ctiles();
    int64_t splits = sm_count() / tiles;
    if (splits < 1) splits = 1;
    if (splits > p.kb_total) splits = p.kb_total;
    if (splits > 32) splits = 32;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    p.splits = (int)((p.kb_total + p.kb_per_split - 1) / p.kb_per_split);
    return p;
}

inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct FwdLayout {
    ColumnSpace cs;
    int n_otiles;
    size_t wimg_bytes;
};
inline FwdLayout fwd_layout(const LayerShape& s, bool has_base) {
    FwdLayout L;
    L.cs = column_space(s.I, has_base);
    L.n_otiles = (s.O + BLOCK_N - 1) / BLOCK_N;
    L.wimg_bytes = (size_t)L.n_otiles * L.cs.kb_total() * 2 * TILE_B_BYTES;
    return L;
}

struct BwdLayout {
    BwdPlan plan;
    size_t dyimg_bytes, partial_bytes;
};
inline BwdLayout bwd_layout(const LayerShape& s, bool has_base) {
    BwdLayout L;
    L.plan = plan_bwd(s, has_base);
    L.dyimg_bytes = (size_t)L.plan.kb_total * L.plan.n_otiles * 2 * BWD_D_SLOT_BYTES;
    L.partial_bytes = (size_t)L.plan.splits * s.O * L.plan.ld_partial() * sizeof(float);
    return L;
}

}  // namespace

bool tc_supported(const LayerShape& s) {
    return s.K >= 1 && s.K <= 3 && s.R() <= RP && s.N >= 1 && s.I >= 1 && s.O >= 1;
}

size_t tc_workspace(int op, const LayerShape& s, bool need_x, bool need_param) {
    // Sized for a layer with a base branch (the larger case).
    if (op == 0) return kWsHeader + align256(fwd_layout(s, true).wimg_bytes);
    size_t b = kWsHeader;
    if (need_param) {
        BwdLayout L = bwd_layout(s, true);
        b += align256(L.dyimg_bytes) + align256(L.partial_bytes);
    }
    (void)need_x;
    return b;
}

cudaError_t tc_forward(int split_terms, const float* x, const float* grid, const float* bw, const float* sw,
                       const float* scaler, float* y, const LayerShape& s,
                       void* ws, size_t ws_bytes, cudaStream_t st) {
    if (s.N == 0) return cudaSuccess;
    const bool has_base = bw != nullptr;
    FwdLayout L = fwd_layout(s, has_base);
    if (!ws || ws_bytes < kWsHeader + L.wimg_bytes) return cudaErrorMemoryAllocation;
    int* status = reinterpret_cast<int*>(ws);
    uint8_t* wimg = reinterpret_cast<uint8_t*>(ws) + kWsHeader;
    const int kb_total = L.cs.kb_total();
    {
        cudaError_t e0 = cudaMemsetAsync(status, 0, sizeof(int), st);
        if (e0 != cudaSuccess) return e0;
        const int64_t chunks = (int64_t)L.n_otiles * kb_total * BLOCK_N * 8;
        int blocks = (int)((chunks + 255) / 256);
        if (blocks > sm_count() * 16) blocks = sm_count() * 16;
        pack_weights_kernel<<<blocks, 256, 0, st>>>(sw, scaler, bw, wimg, s.O, s.I, s.R(), L.cs.kb_spline,
                                                    kb_total, L.n_otiles);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    const int64_t n_mtiles = (s.N + BLOCK_M - 1) / BLOCK_M;
    const int64_t n_tiles = n_mtiles * L.n_otiles;
    int blocks = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
    const int vec_ok = ((s.I & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    cudaError_t e = cudaSuccess;
#define KAN_FWD(KK, NT)                                                                                        \
    do {                                                                                                       \
        e = cudaFuncSetAttribute(tc_forward_kernel<KK, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                 (int)FWD_SMEM_BYTES);                                                         \
        if (e == cudaSuccess)                                                                                  \
            tc_forward_kernel<KK, NT><<<blocks, FWD_THREADS, FWD_SMEM_BYTES, st>>>(                            \
                x, grid, wimg, y, status, s.N, s.I, s.O, s.G, L.cs.kb_spline, kb_total, L.n_otiles, n_tiles,   \
                vec_ok);                                                                                       \
    } while (0)
    if (split_terms == 3) {
        if (s.K == 1) KAN_FWD(1, 3); else if (s.K == 2) KAN_FWD(2, 3); else KAN_FWD(3, 3);
    } else {
        if (s.K == 1) KAN_FWD(1, 1); else if (s.K == 2) KAN_FWD(2, 1); else KAN_FWD(3, 1);
    }
#undef KAN_FWD
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

cudaError_t tc_backward(int split_terms, const float* dY, const float* x, const float* grid, const float* bw,
                        const float* sw, const float* scaler, float* gx, float* gbw, float* gsw,
                        float* gscaler, const LayerShape& s, void* ws, size_t ws_bytes, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    const bool has_base = bw != nullptr;
    const bool need_param = gsw || gscaler || (gbw && has_base);
    if (s.N == 0) return simt_backward<float>(dY, x, grid, bw, sw, scaler, gx, gbw, gsw, gscaler, s, nullptr, 0, st);
    if (need_param) {
        BwdLayout L = bwd_layout(s, has_base);
        const size_t need = kWsHeader + align256(L.dyimg_bytes) + L.partial_bytes;
        if (!ws || ws_bytes < need) return cudaErrorMemoryAllocation;
        int* status = reinterpret_cast<int*>(ws);
        uint8_t* dyimg = reinterpret_cast<uint8_t*>(ws) + kWsHeader;
        float* partial = reinterpret_cast<float*>(dyimg + align256(L.dyimg_bytes));
        {
            if ((e = cudaMemsetAsync(status, 0, sizeof(int), st)) != cudaSuccess) return e;
            const int64_t chunks = L.plan.kb_total * L.plan.n_otiles * 2 * 64 * 16;
            int blocks = (int)((chunks + 255) / 256 < (int64_t)sm_count() * 16 ? (chunks + 255) / 256
                                                                                : (int64_t)sm_count() * 16);
            pack_grad_out_kernel<<<blocks, 256, 0, st>>>(dY, dyimg, s.N, s.O, L.plan.kb_total, L.plan.n_otiles * 2);
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        const int64_t items = L.plan.n_items();
        const int blocks = (int)(items < sm_count() ? items : sm_count());
        const int vec_ok = ((s.I & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
#define KAN_BWD(KK, NT)                                                                                        \
    do {                                                                                                       \
        e = cudaFuncSetAttribute(tc_bwd_param_kernel<KK, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                 (int)BWD_SMEM_BYTES);                                                         \
        if (e == cudaSuccess)                                                                                  \
            tc_bwd_param_kernel<KK, NT><<<blocks, BWD_THREADS, BWD_SMEM_BYTES, st>>>(                          \
                x, grid, dyimg, partial, status, s.N, s.I, s.O, s.G, L.plan, vec_ok);                          \
    } while (0)
        if (split_terms == 3) {
            if (s.K == 1) KAN_BWD(1, 3); else if (s.K == 2) KAN_BWD(2, 3); else KAN_BWD(3, 3);
        } else {
            if (s.K == 1) KAN_BWD(1, 1); else if (s.K == 2) KAN_BWD(2, 1); else KAN_BWD(3, 1);
        }
#undef KAN_BWD
        if (e != cudaSuccess) return e;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        const int64_t ld = L.plan.ld_partial();
        e = finalize_param_grads<float>(partial, L.plan.splits, (int64_t)s.O * ld, ld, RP,
                                        (int64_t)L.plan.ct_spline * BLOCK_N, 1, sw, scaler, gsw, gscaler,
                                        has_base ? gbw : nullptr, s.O, s.I, s.R(), st);
        if (e != cudaSuccess) return e;
    }
    if (gx) {
        // Input gradient: gather formulation on the FMA pipes.
        e = simt_backward<float>(dY, x, grid, bw, sw, scaler, gx, nullptr, nullptr, nullptr, s, nullptr, 0, st);
    }
    return e;
}

}  // namespace kanb200
