// Tensor-core (tcgen05 / TMEM) kernels of the KANLinear path for fp32 tensors.
//
// The spline contraction  y[n,o] = sum_{i,r} B_r(x[n,i]) W_eff[o,i,r] + sum_i silu(x[n,i]) bw[o,i]
// is a dense GEMM whose left operand is never stored: its tiles are evaluated
// from x in registers and written straight into the shared-memory operand
// layout the MMA unit reads.  fp32 accuracy is kept on 16-bit tensor-core
// inputs by splitting every operand value v into hi = bf16(v) and
// lo = bf16(v - hi) and issuing three MMAs per step (hi*hi + lo*hi + hi*lo).
// The tensor-core accumulator truncates on every accumulation, so a long
// reduction is cut into chunks: after a bounded number of k-blocks the TMEM
// accumulator is drained and added, in fp32 with round-to-nearest, to the
// running result in global memory (which stays in L2).
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
// Both contraction kernels are persistent and warp-specialised: 16 worker warps
// (they evaluate the generated operand and, between chunks, drain the
// accumulator), one MMA-issuing thread and one bulk-copy thread.  Every wait is
// bounded.
#include "kan_device.cuh"
#include "kan_tc_common.cuh"

namespace kanb200 {

namespace {

using namespace ptx;

__global__ void build_poly_table_kernel(const float* __restrict__ grid, float* __restrict__ tab,
                                        int I, int G, int K, TabInfo ti) {
    const int nk = ti.nk, R = G + K;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= I * (nk + 1)) return;
    const int f = idx / (nk + 1), e = idx - f * (nk + 1);
    const float* t = grid + (size_t)f * nk;
    float* out = tab + (size_t)f * ti.fs;
    if (e == nk) {                             // header + knot block
        float differs = 0.0f;
        for (int q = 0; q < nk; ++q)
            if (t[q] != grid[q]) differs = 1.0f;
        out[0] = differs;
        out[1] = out[2] = out[3] = 0.0f;
        if (nk <= TAB_FAST_MAX_KNOTS) {
            poly_table_knots12(t, nk, out + 4);
        } else {
            for (int q = 0; q < nk; ++q) out[4 + q] = t[q];
            for (int q = 4 + nk; q < ti.es; ++q) out[q] = 0.0f;
        }
        return;
    }
    poly_table_entry(t, nk, K, R, e, out + ti.es + e * TAB_ENTRY_FLOATS);
}

// ---------------------------------------------------------------------------
// Weight images.  For every (o-tile of 256, k-block of 64 columns) the image
// holds two 32-KB tiles (hi, lo) that are byte-for-byte the shared-memory
// contents the MMA unit expects: 256 rows (outputs) x 128 B (64 columns),
// 128-byte swizzle.  One bulk copy brings a tile in.
// ---------------------------------------------------------------------------
struct ColumnSpace {
    int kb_spline;     // k-blocks (64 columns = 8 chunks of 8 slots) of the spline part
    int kb_base;       // k-blocks (64 features) of the base part, 0 without base
    int kb_total() const { return kb_spline + kb_base; }
};

inline ColumnSpace column_space(int I, int cpf, bool has_base) {
    ColumnSpace c;
    c.kb_spline = (I * cpf + 7) / 8;
    c.kb_base = has_base ? (I + 63) / 64 : 0;
    return c;
}

__global__ void pack_weights_kernel(const float* __restrict__ sw, const float* __restrict__ scaler,
                                    const float* __restrict__ bw, uint8_t* __restrict__ img,
                                    int O, int I, int R, int cpf, int kb_spline, int kb_total, int n_otiles) {
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
                const int g = kb * 8 + cc;                  // chunk -> (feature, 8 of its slots)
                const int f = g / cpf, r0 = (g - f * cpf) * 8;
                if (f < I) {
                    const size_t oi = (size_t)o * I + f;
                    const float sc = scaler ? scaler[oi] : 1.0f;
                    for (int e = 0; e < 8; ++e)
                        if (r0 + e < R) {
                            const float v = sw[oi * R + r0 + e];
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
__global__ void pack_grad_out_kernel(const float* __restrict__ dY, int64_t ldy, uint8_t* __restrict__ img,
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
            const float* p = dY + (size_t)n * ldy + o0;
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
// Common geometry of the two contraction kernels
// ---------------------------------------------------------------------------
constexpr int WORKER_WARPS = 16;                       // operand producers + accumulator drain
constexpr int WORKER_THREADS = WORKER_WARPS * 32;
constexpr int TC_THREADS = (WORKER_WARPS + 2) * 32;    // + MMA warp + bulk-copy warp
constexpr int MMA_WARP = WORKER_WARPS;              // warp MMA_WARP + 1 issues the bulk copies

// Fire-and-forget float32 add of four consecutive values, performed in L2 (IEEE round-to-nearest).
// The running result is never read back by the SM, so a drain costs no load latency.  An element
// is only ever touched by ONE thread, in program order (a store for the first chunk, then adds), so
// the sum is the same bits on every run.
__device__ __forceinline__ void red_add_v4(float* dst, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

// Adds (or, for the first chunk, stores) 32 accumulator columns of one row.
__device__ __forceinline__ void drain_row32(float* __restrict__ dst, const uint32_t (&r)[32], bool first,
                                            int valid, bool vec) {
    if (vec && valid >= 32) {
        if (first) {
            float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                d4[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                    __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                red_add_v4(dst + 4 * q, __uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                           __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        }
    } else {
#pragma unroll
        for (int q = 0; q < 32; ++q)
            if (q < valid) dst[q] = first ? __uint_as_float(r[q]) : dst[q] + __uint_as_float(r[q]);
    }
}

// The same for the 32 rows of a warp at once, with full 128-byte lines per request: after a load of
// tensor memory lane l holds 32 columns of row l, so a store or reduction per lane touches 16 bytes in
// each of 32 rows.  Three butterfly exchanges (lane bit 2 + t <-> slot bit t) re-sort the 8 groups of 4
// columns so that slot q of lane 4 b + a holds columns 4b .. 4b+3 of row 4 q + a; every instruction then
// covers four rows with 128 contiguous bytes each (measured on the whole y of 65536 x 1024: 2.36 against
// 1.32 TB/s of reductions).  All 32 rows and columns must be valid and 16-byte aligned.
__device__ __forceinline__ void drain_rows32_warp(float* __restrict__ warp_dst, size_t ld, uint32_t (&r)[32], int lane,
                                                  bool first) {
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int lane_bit = 4 << t, slot_bit = 1 << t;
        const bool up = (lane & lane_bit) != 0;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (s & slot_bit) continue;
            const int s2 = s | slot_bit;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t send = up ? r[4 * s + w] : r[4 * s2 + w];
                const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, lane_bit);
                if (up) r[4 * s + w] = recv;
                else r[4 * s2 + w] = recv;
            }
        }
    }
    float* dst = warp_dst + (size_t)(lane & 3) * ld + 4 * (lane >> 2);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        float* d = dst + (size_t)(4 * q) * ld;
        if (first)
            *reinterpret_cast<float4*>(d) = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                        __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        else
            red_add_v4(d, __uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                       __uint_as_float(r[4 * q + 3]));
    }
}

// ---------------------------------------------------------------------------
// Forward kernel:  y[n, o] = sum_c A[n, c] W[o, c]
// ---------------------------------------------------------------------------
// Tile = 128 samples x up to 512 outputs (one or two 256-wide sub-tiles sharing
// the generated A tile; all 512 TMEM columns).  A stage = 128 x 64 bf16 hi + lo.
constexpr int FWD_A_STAGES = 2, FWD_B_SLOTS = 5;
constexpr uint32_t FWD_A_STAGE_BYTES = 2 * TILE_A_BYTES;                  // hi + lo
constexpr uint32_t FWD_SMEM_A = 0;
constexpr uint32_t FWD_SMEM_B = FWD_SMEM_A + FWD_A_STAGES * FWD_A_STAGE_BYTES;
constexpr uint32_t FWD_SMEM_CTRL = FWD_SMEM_B + FWD_B_SLOTS * TILE_B_BYTES;
constexpr uint32_t FWD_CTRL_BYTES = 256 + TAB_SMEM_FLOATS * 4;   // barriers + the shared-grid table
constexpr uint32_t FWD_SMEM_BYTES = FWD_SMEM_CTRL + FWD_CTRL_BYTES;
static_assert(FWD_SMEM_BYTES <= 232448, "forward kernel shared memory exceeds 227 KB");

struct FwdCtrl {
    uint64_t fullA[5], emptyA[5];          // sized for both forward kernels
    uint64_t fullB[6], emptyB[6];
    // per 256-column accumulator: its chain is complete / its columns have been drained.  Kept apart
    // so that one accumulator is drained while the MMAs of the other run.
    uint64_t chunkFull[2], drained[2];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(FwdCtrl) <= 256, "control block too large");

struct FwdParams {
    int64_t N;
    int I, O, G;
    int kb_spline, kb_total;
    int n_otiles, n_opairs;
    int64_t n_tiles;
    int chunk_kb;          // k-blocks accumulated in TMEM between drains
    int vec_x, vec_x2, vec_y;
    // Few row tiles (small batches): every chain of chunk_kb blocks is a work item of its own
    // (item = tile * n_ksplit + chain) and stores its result in slab[chain][N][O]; a second kernel adds
    // the slabs in fixed order.  n_ksplit == 1: an item is a whole tile and accumulates in y itself.
    int n_ksplit;
    float* slab;
    TabInfo ti;
    __host__ __device__ int64_t n_items() const { return n_tiles * n_ksplit; }
};

// item -> tile, blocks [kb0, kb1) and destination of the item's result
__device__ __forceinline__ void fwd_item(const FwdParams& P, int64_t item, float* y, int64_t& tile, int& kb0, int& kb1,
                                         float*& dst) {
    if (P.n_ksplit > 1) {
        tile = item / P.n_ksplit;
        const int chain = (int)(item - tile * P.n_ksplit);
        kb0 = chain * P.chunk_kb;
        kb1 = kb0 + P.chunk_kb < P.kb_total ? kb0 + P.chunk_kb : P.kb_total;
        dst = P.slab + (size_t)chain * (size_t)P.N * P.O;
    } else {
        tile = item;
        kb0 = 0;
        kb1 = P.kb_total;
        dst = y;
    }
}

template <int NTERMS, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_forward_kernel(const float* __restrict__ x, const float* __restrict__ tab, const uint8_t* __restrict__ wimg,
                  float* __restrict__ y, int* __restrict__ status, const FwdParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    FwdCtrl* ctrl = reinterpret_cast<FwdCtrl*>(smem + FWD_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + FWD_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool shared_grid = grid_is_shared(tab, P.I, P.ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < P.ti.fs) stab[threadIdx.x] = tab[threadIdx.x];

    if ((sbase & 1023u) != 0) {                 // swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) report_status(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < FWD_A_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullA[s]), WORKER_THREADS);
            mbar_init(smem_u32(&ctrl->emptyA[s]), 1);
        }
        for (int s = 0; s < FWD_B_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullB[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyB[s]), 1);
        }
        for (int j = 0; j < 2; ++j) {
            mbar_init(smem_u32(&ctrl->chunkFull[j]), 1);
            mbar_init(smem_u32(&ctrl->drained[j]), WORKER_THREADS);
        }
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp < WORKER_WARPS) {
        // ===== workers: x -> basis / silu -> swizzled A tile; drain between chunks =====
        const int quad = warp & 3;                        // TMEM lane quadrant = row group
        const int part = warp >> 2;                       // which quarter of the k-block / column groups
        const int row = quad * 32 + lane;
        uint32_t it = 0, n_drained[2] = {0, 0};
        bool ok = true;
        // drain bookkeeping: the chunk that ended most recently and is not yet added to y
        bool pend = false, pend_first = false;
        int64_t pend_mt = 0;
        int pend_op = 0;
        float* pend_dst = y;

        auto drain = [&]() -> bool {
            const int64_t n = pend_mt * BLOCK_M + row;
            const int nsub = (P.n_otiles - 2 * pend_op) >= 2 ? 2 : 1;
#pragma unroll 1
            for (int j = 0; j < nsub; ++j) {
                if (!mbar_wait(smem_u32(&ctrl->chunkFull[j]), n_drained[j] & 1u, abort_flag)) return false;
                ++n_drained[j];
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = part; c < BLOCK_N / 32; c += 4) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + j * BLOCK_N + c * 32, r);
                    tmem_ld_wait();
                    const int col0 = (pend_op * 2 + j) * BLOCK_N + c * 32;
                    const int64_t n0 = n - lane;                   // first of the warp's 32 rows
                    if (P.vec_y && n0 + 32 <= P.N && col0 + 32 <= P.O)        // uniform over the warp
                        drain_rows32_warp(pend_dst + (size_t)n0 * P.O + col0, (size_t)P.O, r, lane, pend_first);
                    else if (n < P.N && col0 < P.O)
                        drain_row32(pend_dst + (size_t)n * P.O + col0, r, pend_first, P.O - col0, P.vec_y != 0);
                }
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&ctrl->drained[j]));
            }
            pend = false;
            return true;
        };

        for (int64_t item = blockIdx.x; item < P.n_items() && ok; item += gridDim.x) {
            int64_t tile;
            int kb0, kb1;
            float* dst;
            fwd_item(P, item, y, tile, kb0, kb1, dst);
            const int64_t mt = tile / P.n_opairs;
            const int op = (int)(tile - mt * P.n_opairs);
            const int64_t n = mt * BLOCK_M + row;
            const bool row_ok = n < P.N;
            const float* xrow = x + (size_t)(row_ok ? n : 0) * P.I;
            // A thread fills chunks g0 = 8 kb + 2 part and g0 + 1 of the k-block; chunk g belongs to
            // feature g / cpf and holds its slots 8 (g % cpf) ..  The inputs of the next k-block
            // are loaded one iteration ahead.
            const int cpf = WIDE ? P.ti.cpf : 1;
            float nx0 = 0.f, nx1 = 0.f;
            auto chunk_pair = [&](int kb, int& f0, int& cw0, int& f1, int& cw1) {
                const int g0 = kb * 8 + part * 2;
                if (!WIDE) {
                    f0 = g0; cw0 = 0; f1 = g0 + 1; cw1 = 0;
                } else {
                    f0 = g0 / cpf; cw0 = g0 - f0 * cpf;
                    f1 = f0; cw1 = cw0 + 1;
                    if (cw1 == cpf) { f1 = f0 + 1; cw1 = 0; }
                }
            };
            auto prefetch_spline = [&](int kb) {
                int f0, cw0, f1, cw1;
                chunk_pair(kb, f0, cw0, f1, cw1);
                if (!WIDE && P.vec_x2 && row_ok && f0 + 1 < P.I) {
                    const float2 v = __ldg(reinterpret_cast<const float2*>(xrow + f0));
                    nx0 = v.x;
                    nx1 = v.y;
                } else {
                    nx0 = (row_ok && f0 < P.I) ? __ldg(xrow + f0) : 0.f;
                    nx1 = (row_ok && f1 < P.I) ? __ldg(xrow + f1) : 0.f;
                }
            };
            if (kb0 < P.kb_spline) prefetch_spline(kb0);
            // position inside the chain, kept as a counter (kb0 starts a chain): a division per block in
            // each of the 512 workers is a measurable share of their instruction stream
            int in_chain = 0;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t stage = it % FWD_A_STAGES;
                const uint32_t a_hi = sbase + FWD_SMEM_A + stage * FWD_A_STAGE_BYTES;
                const uint32_t a_lo = a_hi + TILE_A_BYTES;
                const bool chunk_start = in_chain == 0;
                if (kb < P.kb_spline) {
                    int f0, cw0, f1, cw1;
                    chunk_pair(kb, f0, cw0, f1, cw1);
                    const float x0 = nx0, x1 = nx1;
                    if (kb + 1 < P.kb_spline) prefetch_spline(kb + 1);
                    const bool ok0 = row_ok && f0 < P.I, ok1 = row_ok && f1 < P.I;
                    // features beyond I read the last feature's table; their rows are zeroed below
                    const float* t0 = tab + (size_t)(f0 < P.I ? f0 : P.I - 1) * P.ti.fs;
                    const float* t1 = tab + (size_t)(f1 < P.I ? f1 : P.I - 1) * P.ti.fs;
                    uint4 hi0, lo0, hi1, lo1;
                    Window w = shared_grid ? eval_window<SPLIT, true, WIDE>(stab, P.ti, x0)
                                           : eval_window<SPLIT, false, WIDE>(t0, P.ti, x0);
                    place_window<SPLIT>(w, cw0, hi0, lo0);
                    if (!WIDE || f1 != f0)                 // uniform over the warp
                        w = shared_grid ? eval_window<SPLIT, true, WIDE>(stab, P.ti, x1)
                                        : eval_window<SPLIT, false, WIDE>(t1, P.ti, x1);
                    place_window<SPLIT>(w, cw1, hi1, lo1);
                    if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / FWD_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint4 zero = make_uint4(0, 0, 0, 0);
                    const uint32_t off0 = sw128_chunk_offset((uint32_t)row, (uint32_t)(part * 2));
                    const uint32_t off1 = sw128_chunk_offset((uint32_t)row, (uint32_t)(part * 2 + 1));
                    st_shared_v4(a_hi + off0, ok0 ? hi0 : zero);
                    st_shared_v4(a_hi + off1, ok1 ? hi1 : zero);
                    if (SPLIT) {
                        st_shared_v4(a_lo + off0, ok0 ? lo0 : zero);
                        st_shared_v4(a_lo + off1, ok1 ? lo1 : zero);
                    }
                } else {
                    const int f0 = (kb - P.kb_spline) * 64 + part * 16;
                    float xv[2][8];
                    load_x8(x, n, row_ok, P.I, f0, P.vec_x != 0, xv[0]);
                    load_x8(x, n, row_ok, P.I, f0 + 8, P.vec_x != 0, xv[1]);
                    if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / FWD_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint4 hi, lo;
                        silu_chunk<SPLIT>(xv[c], hi, lo);
                        const uint32_t off = sw128_chunk_offset((uint32_t)row, (uint32_t)(part * 2 + c));
                        st_shared_v4(a_hi + off, hi);
                        if (SPLIT) st_shared_v4(a_lo + off, lo);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullA[stage]));
                // The previous chunk is drained only after the first k-block of the next one has
                // been produced, so the MMA pipe restarts without waiting for the producers.
                if (pend && chunk_start) {
                    if (!drain()) {
                        ok = false;
                        break;
                    }
                }
                if (++in_chain == P.chunk_kb) in_chain = 0;
                if (in_chain == 0 || kb + 1 == kb1) {
                    pend = true;
                    pend_first = P.n_ksplit > 1 || kb < P.chunk_kb;
                    pend_mt = mt;
                    pend_op = op;
                    pend_dst = dst;
                }
            }
        }
        if (ok && pend) drain();
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // ===== MMA issue =====
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, false, false);
            constexpr uint64_t dbase = make_sdesc_sw128(16, 1024);
            uint32_t it = 0, bslot = 0, n_chunks[2] = {0, 0};
            bool ok = true;
            for (int64_t item = blockIdx.x; item < P.n_items() && ok; item += gridDim.x) {
                int64_t tile;
                int kb0, kb1;
                float* dst;
                fwd_item(P, item, y, tile, kb0, kb1, dst);
                const int64_t mt = tile / P.n_opairs;
                const int op = (int)(tile - mt * P.n_opairs);
                const int nsub = (P.n_otiles - 2 * op) >= 2 ? 2 : 1;
                int in_chain = 0;
                for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
                    const uint32_t stage = it % FWD_A_STAGES;
                    const uint32_t a_hi = sbase + FWD_SMEM_A + stage * FWD_A_STAGE_BYTES;
                    const uint32_t a_lo = a_hi + TILE_A_BYTES;
                    const bool chunk_start = in_chain == 0;
                    if (++in_chain == P.chunk_kb) in_chain = 0;
                    const bool chunk_end = in_chain == 0 || kb + 1 == kb1;
                    if (!mbar_wait(smem_u32(&ctrl->fullA[stage]), (it / FWD_A_STAGES) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    for (int j = 0; j < nsub && ok; ++j) {
                        const uint32_t d_tmem = tmem_base + j * BLOCK_N;
                        if (chunk_start && n_chunks[j] > 0) {
                            // this accumulator may be overwritten only after the workers have drained it
                            if (!mbar_wait(smem_u32(&ctrl->drained[j]), (n_chunks[j] - 1) & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                        }
                        const uint32_t slot_h = bslot % FWD_B_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->fullB[slot_h]), (bslot / FWD_B_SLOTS) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t b_hi = sbase + FWD_SMEM_B + slot_h * TILE_B_BYTES;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, a_hi + ks * 32), sdesc_at(dbase, b_hi + ks * 32),
                                       idesc, (!chunk_start || ks > 0) ? 1u : 0u);
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
                            if (!mbar_wait(smem_u32(&ctrl->fullB[slot_l]), (bslot / FWD_B_SLOTS) & 1u, abort_flag)) {
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
                        if (chunk_end) {
                            // this accumulator's chain is complete: its drain overlaps the MMAs of the other
                            mma_commit(smem_u32(&ctrl->chunkFull[j]));
                            ++n_chunks[j];
                        }
                    }
                    if (!ok) break;
                    mma_commit(smem_u32(&ctrl->emptyA[stage]));
                }
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk-copy producer for weight tiles =====
            uint32_t bslot = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < P.n_items() && ok; item += gridDim.x) {
                int64_t tile;
                int kb0, kb1;
                float* dst;
                fwd_item(P, item, y, tile, kb0, kb1, dst);
                const int64_t mt = tile / P.n_opairs;
                const int op = (int)(tile - mt * P.n_opairs);
                const int nsub = (P.n_otiles - 2 * op) >= 2 ? 2 : 1;
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    for (int j = 0; j < nsub && ok; ++j) {
                        const uint8_t* src = wimg + ((size_t)(2 * op + j) * P.kb_total + kb) * (2 * (size_t)TILE_B_BYTES);
                        for (int term = 0; term < (SPLIT ? 2 : 1); ++term, ++bslot) {
                            const uint32_t slot = bslot % FWD_B_SLOTS;
                            if (!mbar_wait(smem_u32(&ctrl->emptyB[slot]), ((bslot / FWD_B_SLOTS) & 1u) ^ 1u,
                                           abort_flag)) {
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
    }

    // ===== teardown =====
    if (*abort_flag) {
        if (lane == 0) report_status(status, kStatusTimeout);
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
// Forward kernel with the generated operand in TENSOR MEMORY.
// The workers store their rows of A straight into tensor memory (tcgen05.st; lane = sample row, one
// 32-bit column = two consecutive K elements), the MMA takes A from there (no shared-memory read
// for it), and shared memory only carries the weight tiles.  Tile = 128 samples x 256 outputs (one
// accumulator of 256 columns; four operand stages of 64 columns fill the rest), so every generated
// tile serves 256 outputs instead of the 512 of the kernel above: it is the faster kernel for
// layers of up to 256 outputs (measured, 8192 rows: 784 -> 256 0.216 against 0.229 ms, 256 -> 10
// 0.077 against 0.087 ms) and the slower one beyond (1024 -> 1024 at 65536 rows: 3.9 against 2.9 ms:
// twice the operand production and twice the weight-tile traffic per output).
// ---------------------------------------------------------------------------
constexpr int FTS_A_STAGES = 4, FTS_B_SLOTS = 6;                 // one operand stage per group of 4 worker warps
static_assert(FTS_A_STAGES * 4 == WORKER_WARPS, "one operand stage per worker group");
constexpr uint32_t FTS_TMEM_A = 256;
constexpr uint32_t FTS_SMEM_B = 0;
constexpr uint32_t FTS_SMEM_CTRL = FTS_SMEM_B + FTS_B_SLOTS * TILE_B_BYTES;
constexpr uint32_t FTS_SMEM_BYTES = FTS_SMEM_CTRL + FWD_CTRL_BYTES;
static_assert(FTS_SMEM_BYTES <= 232448, "forward kernel shared memory exceeds 227 KB");

template <int NTERMS, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_forward_ts_kernel(const float* __restrict__ x, const float* __restrict__ tab, const uint8_t* __restrict__ wimg,
                  float* __restrict__ y, int* __restrict__ status, const FwdParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    FwdCtrl* ctrl = reinterpret_cast<FwdCtrl*>(smem + FTS_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + FTS_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool shared_grid = grid_is_shared(tab, P.I, P.ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < P.ti.fs) stab[threadIdx.x] = tab[threadIdx.x];

    if ((sbase & 1023u) != 0) {                 // swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) report_status(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < FTS_A_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullA[s]), WORKER_THREADS / FTS_A_STAGES);     // one group of worker warps
            mbar_init(smem_u32(&ctrl->emptyA[s]), 1);
        }
        for (int s = 0; s < FTS_B_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullB[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyB[s]), 1);
        }
        for (int j = 0; j < 2; ++j) {
            mbar_init(smem_u32(&ctrl->chunkFull[j]), 1);
            mbar_init(smem_u32(&ctrl->drained[j]), WORKER_THREADS);
        }
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp < WORKER_WARPS) {
        // ===== workers: x -> basis / silu -> swizzled A tile; drain between chunks =====
        const int quad = warp & 3;                        // TMEM lane quadrant = row group
        const int part = warp >> 2;                       // which quarter of the k-block / column groups
        const int row = quad * 32 + lane;
        uint32_t it = 0, n_drained[2] = {0, 0};
        bool ok = true;
        // drain bookkeeping: the chunk that ended most recently and is not yet added to y
        bool pend = false, pend_first = false;
        int64_t pend_mt = 0;
        int pend_op = 0;
        float* pend_dst = y;

        auto drain = [&]() -> bool {
            const int64_t n = pend_mt * BLOCK_M + row;
#pragma unroll 1
            for (int j = 0; j < 1; ++j) {
                if (!mbar_wait(smem_u32(&ctrl->chunkFull[j]), n_drained[j] & 1u, abort_flag)) return false;
                ++n_drained[j];
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = part; c < BLOCK_N / 32; c += 4) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + j * BLOCK_N + c * 32, r);
                    tmem_ld_wait();
                    const int col0 = pend_op * BLOCK_N + c * 32;
                    const int64_t n0 = n - lane;                   // first of the warp's 32 rows
                    if (P.vec_y && n0 + 32 <= P.N && col0 + 32 <= P.O)        // uniform over the warp
                        drain_rows32_warp(pend_dst + (size_t)n0 * P.O + col0, (size_t)P.O, r, lane, pend_first);
                    else if (n < P.N && col0 < P.O)
                        drain_row32(pend_dst + (size_t)n * P.O + col0, r, pend_first, P.O - col0, P.vec_y != 0);
                }
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&ctrl->drained[j]));
            }
            pend = false;
            return true;
        };

        for (int64_t item = blockIdx.x; item < P.n_items() && ok; item += gridDim.x) {
            int64_t tile;
            int kb0, kb1;
            float* dst;
            fwd_item(P, item, y, tile, kb0, kb1, dst);
            const int64_t mt = tile / P.n_otiles;
            const int op = (int)(tile - mt * P.n_otiles);          // the 256-output tile
            const int64_t n = mt * BLOCK_M + row;
            const bool row_ok = n < P.N;
            const float* xrow = x + (size_t)(row_ok ? n : 0) * P.I;
            // The four groups of four worker warps take the k-blocks in turn: group g fills operand stage
            // g with every fourth block (block counter it = g mod 4), a thread = one row of it, all eight
            // chunks (chunk c of block kb is global chunk g = 8 kb + c; it belongs to feature g / cpf and
            // holds its slots 8 (g % cpf) ..).  Four blocks are therefore in production at any time, and a
            // thread has eight independent window evaluations to overlap.
            const int cpf = WIDE ? P.ti.cpf : 1;
            auto chunk_pair = [&](int kb, int p, int& f0, int& cw0, int& f1, int& cw1) {
                const int g0 = kb * 8 + p * 2;
                if (!WIDE) {
                    f0 = g0; cw0 = 0; f1 = g0 + 1; cw1 = 0;
                } else {
                    f0 = g0 / cpf; cw0 = g0 - f0 * cpf;
                    f1 = f0; cw1 = cw0 + 1;
                    if (cw1 == cpf) { f1 = f0 + 1; cw1 = 0; }
                }
            };
            int in_chain = 0;                                      // position inside the chain (kb0 starts one)
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t stage = it % FTS_A_STAGES;
                const bool chunk_start = in_chain == 0;
                if ((int)stage == part) {
                    // operand stage in tensor memory: 32 columns of bf16 pairs (hi), then 32 (lo)
                    const uint32_t a_hi = tmem_base + ((uint32_t)(quad * 32) << 16) + FTS_TMEM_A + stage * 64;
                    const uint32_t a_lo = a_hi + 32;
                    float xb[8];
                    if (kb < P.kb_spline && !WIDE) load_x8(x, n, row_ok, P.I, kb * 8, P.vec_x != 0, xb);
                    if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / FTS_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if (kb < P.kb_spline) {
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            int f0, cw0, f1, cw1;
                            chunk_pair(kb, p, f0, cw0, f1, cw1);
                            float x0, x1;
                            if (!WIDE) {
                                x0 = xb[2 * p];
                                x1 = xb[2 * p + 1];
                            } else {
                                x0 = (row_ok && f0 < P.I) ? __ldg(xrow + f0) : 0.f;
                                x1 = (row_ok && f1 < P.I) ? __ldg(xrow + f1) : 0.f;
                            }
                            const bool ok0 = row_ok && f0 < P.I, ok1 = row_ok && f1 < P.I;
                            // features beyond I read the last feature's table; their rows are zeroed below
                            const float* t0 = tab + (size_t)(f0 < P.I ? f0 : P.I - 1) * P.ti.fs;
                            const float* t1 = tab + (size_t)(f1 < P.I ? f1 : P.I - 1) * P.ti.fs;
                            uint4 hi0, lo0, hi1, lo1;
                            Window w = shared_grid ? eval_window<SPLIT, true, WIDE>(stab, P.ti, x0)
                                                   : eval_window<SPLIT, false, WIDE>(t0, P.ti, x0);
                            place_window<SPLIT>(w, cw0, hi0, lo0);
                            if (!WIDE || f1 != f0)                 // uniform over the warp
                                w = shared_grid ? eval_window<SPLIT, true, WIDE>(stab, P.ti, x1)
                                                : eval_window<SPLIT, false, WIDE>(t1, P.ti, x1);
                            place_window<SPLIT>(w, cw1, hi1, lo1);
                            const uint4 zero = make_uint4(0, 0, 0, 0);
                            if (!ok0) { hi0 = zero; lo0 = zero; }
                            if (!ok1) { hi1 = zero; lo1 = zero; }
                            {
                                const uint32_t wd[8] = {hi0.x, hi0.y, hi0.z, hi0.w, hi1.x, hi1.y, hi1.z, hi1.w};
                                tmem_st_32x8(a_hi + p * 8, wd);
                            }
                            if (SPLIT) {
                                const uint32_t wd[8] = {lo0.x, lo0.y, lo0.z, lo0.w, lo1.x, lo1.y, lo1.z, lo1.w};
                                tmem_st_32x8(a_lo + p * 8, wd);
                            }
                        }
                    } else {
#pragma unroll 1
                        for (int p = 0; p < 4; ++p) {
                            const int f0 = (kb - P.kb_spline) * 64 + p * 16;
                            float xv[2][8];
                            load_x8(x, n, row_ok, P.I, f0, P.vec_x != 0, xv[0]);
                            load_x8(x, n, row_ok, P.I, f0 + 8, P.vec_x != 0, xv[1]);
                            uint4 hi[2], lo[2];
                            silu_chunk<SPLIT>(xv[0], hi[0], lo[0]);
                            silu_chunk<SPLIT>(xv[1], hi[1], lo[1]);
                            {
                                const uint32_t wd[8] = {hi[0].x, hi[0].y, hi[0].z, hi[0].w,
                                                        hi[1].x, hi[1].y, hi[1].z, hi[1].w};
                                tmem_st_32x8(a_hi + p * 8, wd);
                            }
                            if (SPLIT) {
                                const uint32_t wd[8] = {lo[0].x, lo[0].y, lo[0].z, lo[0].w,
                                                        lo[1].x, lo[1].y, lo[1].z, lo[1].w};
                                tmem_st_32x8(a_lo + p * 8, wd);
                            }
                        }
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                    mbar_arrive(smem_u32(&ctrl->fullA[stage]));
                }
                // The previous chunk is drained only after the first k-block of the next one has
                // been produced, so the MMA pipe restarts without waiting for the producers.
                if (pend && chunk_start) {
                    if (!drain()) {
                        ok = false;
                        break;
                    }
                }
                if (++in_chain == P.chunk_kb) in_chain = 0;
                if (in_chain == 0 || kb + 1 == kb1) {
                    pend = true;
                    pend_first = P.n_ksplit > 1 || kb < P.chunk_kb;
                    pend_mt = mt;
                    pend_op = op;
                    pend_dst = dst;
                }
            }
        }
        if (ok && pend) drain();
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // ===== MMA issue =====
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, false, false);
            constexpr uint64_t dbase = make_sdesc_sw128(16, 1024);
            uint32_t it = 0, bslot = 0, n_chunks[2] = {0, 0};
            bool ok = true;
            for (int64_t item = blockIdx.x; item < P.n_items() && ok; item += gridDim.x) {
                int64_t tile;
                int kb0, kb1;
                float* dst;
                fwd_item(P, item, y, tile, kb0, kb1, dst);
                const int nsub = 1;
                int in_chain = 0;
                for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
                    const uint32_t stage = it % FTS_A_STAGES;
                    const uint32_t a_hi = tmem_base + FTS_TMEM_A + stage * 64;
                    const uint32_t a_lo = a_hi + 32;
                    const bool chunk_start = in_chain == 0;
                    if (++in_chain == P.chunk_kb) in_chain = 0;
                    const bool chunk_end = in_chain == 0 || kb + 1 == kb1;
                    if (!mbar_wait(smem_u32(&ctrl->fullA[stage]), (it / FTS_A_STAGES) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    for (int j = 0; j < nsub && ok; ++j) {
                        const uint32_t d_tmem = tmem_base + j * BLOCK_N;
                        if (chunk_start && n_chunks[j] > 0) {
                            // this accumulator may be overwritten only after the workers have drained it
                            if (!mbar_wait(smem_u32(&ctrl->drained[j]), (n_chunks[j] - 1) & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                        }
                        const uint32_t slot_h = bslot % FTS_B_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->fullB[slot_h]), (bslot / FTS_B_SLOTS) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t b_hi = sbase + FTS_SMEM_B + slot_h * TILE_B_BYTES;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ts(d_tmem, a_hi + ks * 8, sdesc_at(dbase, b_hi + ks * 32), idesc,
                                       (!chunk_start || ks > 0) ? 1u : 0u);
                        if (SPLIT) {
#pragma unroll
                            for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                                mma_f16_ts(d_tmem, a_lo + ks * 8, sdesc_at(dbase, b_hi + ks * 32), idesc, 1u);
                        }
                        mma_commit(smem_u32(&ctrl->emptyB[slot_h]));
                        ++bslot;
                        if (SPLIT) {
                            const uint32_t slot_l = bslot % FTS_B_SLOTS;
                            if (!mbar_wait(smem_u32(&ctrl->fullB[slot_l]), (bslot / FTS_B_SLOTS) & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t b_lo = sbase + FTS_SMEM_B + slot_l * TILE_B_BYTES;
#pragma unroll
                            for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                                mma_f16_ts(d_tmem, a_hi + ks * 8, sdesc_at(dbase, b_lo + ks * 32), idesc, 1u);
                            mma_commit(smem_u32(&ctrl->emptyB[slot_l]));
                            ++bslot;
                        }
                        if (chunk_end) {
                            // this accumulator's chain is complete: its drain overlaps the MMAs of the other
                            mma_commit(smem_u32(&ctrl->chunkFull[j]));
                            ++n_chunks[j];
                        }
                    }
                    if (!ok) break;
                    mma_commit(smem_u32(&ctrl->emptyA[stage]));
                }
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk-copy producer for weight tiles =====
            uint32_t bslot = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < P.n_items() && ok; item += gridDim.x) {
                int64_t tile;
                int kb0, kb1;
                float* dst;
                fwd_item(P, item, y, tile, kb0, kb1, dst);
                const int64_t mt = tile / P.n_otiles;
                const int op = (int)(tile - mt * P.n_otiles);
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    {
                        const uint8_t* src = wimg + ((size_t)op * P.kb_total + kb) * (2 * (size_t)TILE_B_BYTES);
                        for (int term = 0; term < (SPLIT ? 2 : 1); ++term, ++bslot) {
                            const uint32_t slot = bslot % FTS_B_SLOTS;
                            if (!mbar_wait(smem_u32(&ctrl->emptyB[slot]), ((bslot / FTS_B_SLOTS) & 1u) ^ 1u,
                                           abort_flag)) {
                                ok = false;
                                break;
                            }
                            const uint32_t bar = smem_u32(&ctrl->fullB[slot]);
                            mbar_arrive_expect_tx(bar, TILE_B_BYTES);
                            bulk_g2s(sbase + FTS_SMEM_B + slot * TILE_B_BYTES, src + (size_t)term * TILE_B_BYTES,
                                     TILE_B_BYTES, bar);
                        }
                    }
                }
            }
        }
    }

    // ===== teardown =====
    if (*abort_flag) {
        if (lane == 0) report_status(status, kStatusTimeout);
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
// silu operand is generated by the worker warps.  Every `chunk_kb` blocks of 64
// samples the accumulator is drained into the item's slab of partial sums.
constexpr int BWD_G_STAGES = 2, BWD_D_SLOTS = 3;
constexpr uint32_t BWD_G_STAGE_BYTES = 2 * TILE_B_BYTES;                 // hi + lo, 256 c x 64 n
constexpr uint32_t BWD_D_SLOT_BYTES = 2 * TILE_A_BYTES;                  // hi + lo, 128 o x 64 n
constexpr uint32_t BWD_SMEM_G = 0;
constexpr uint32_t BWD_SMEM_D = BWD_SMEM_G + BWD_G_STAGES * BWD_G_STAGE_BYTES;
constexpr uint32_t BWD_SMEM_CTRL = BWD_SMEM_D + BWD_D_SLOTS * BWD_D_SLOT_BYTES;
constexpr uint32_t BWD_CTRL_BYTES = 256 + TAB_SMEM_FLOATS * 4;   // barriers + the shared-grid table
constexpr uint32_t BWD_SMEM_BYTES = BWD_SMEM_CTRL + BWD_CTRL_BYTES;
static_assert(BWD_SMEM_BYTES <= 232448, "backward kernel shared memory exceeds 227 KB");

struct BwdCtrl {
    uint64_t fullG[BWD_G_STAGES], emptyG[BWD_G_STAGES];
    uint64_t fullD[BWD_D_SLOTS], emptyD[BWD_D_SLOTS];
    uint64_t chunkFull[2], drained[2];     // per 128-row half of the accumulator (see FwdCtrl)
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(BwdCtrl) <= 256, "control block too large");

struct BwdPlan {
    int n_otiles;          // tiles of 256 outputs
    int ct_spline;         // column tiles of 32 chunks (8 slots each) of the spline part
    int ct_base;           // column tiles of 256 base features
    int splits;
    int chunk_kb;          // 64-sample blocks accumulated in TMEM between drains
    int64_t kb_total;      // 64-sample blocks
    int64_t kb_per_split;
    __host__ __device__ int n_ctiles() const { return ct_spline + ct_base; }
    __host__ __device__ int64_t n_items() const { return (int64_t)n_otiles * n_ctiles() * splits; }
    // floats of one split's slab: every (o-tile, c-tile) owns a 256 x 256 block
    __host__ __device__ int64_t slab_floats() const { return (int64_t)n_otiles * n_ctiles() * 256 * 256; }
};

template <int NTERMS, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_bwd_param_kernel(const float* __restrict__ x, const float* __restrict__ tab, const uint8_t* __restrict__ dyimg,
                    float* __restrict__ partial, int* __restrict__ status,
                    int64_t N, int I, int O, BwdPlan plan, TabInfo ti, int vec_ok) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    BwdCtrl* ctrl = reinterpret_cast<BwdCtrl*>(smem + BWD_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + BWD_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool shared_grid = grid_is_shared(tab, I, ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < ti.fs) stab[threadIdx.x] = tab[threadIdx.x];
    const int n_ohalves = plan.n_otiles * 2;
    const int n_ctiles = plan.n_ctiles();
    const int64_t n_items = plan.n_items();

    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) report_status(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < BWD_G_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullG[s]), WORKER_THREADS);
            mbar_init(smem_u32(&ctrl->emptyG[s]), 1);
        }
        for (int s = 0; s < BWD_D_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullD[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyD[s]), 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&ctrl->chunkFull[h]), 1);
            mbar_init(smem_u32(&ctrl->drained[h]), WORKER_THREADS);
        }
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
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
    auto k_range = [&](int sp, int64_t& kb0, int64_t& kb1) {
        kb0 = (int64_t)sp * plan.kb_per_split;
        kb1 = kb0 + plan.kb_per_split;
        if (kb1 > plan.kb_total) kb1 = plan.kb_total;
    };

    if (warp < WORKER_WARPS) {
        // ===== workers: 64 samples x 256 columns per block, MN-major; drain between chunks =====
        const int quad = warp & 3, part = warp >> 2;
        // spline tiles: thread = (sample, 4 chunks); base tiles: thread = (4 samples, 8 features)
        const int n_loc = (warp & 1) * 32 + lane;       // sample within the block (spline tiles)
        const int fq = warp >> 1;                       // group of 4 chunks (spline tiles)
        const int kg = warp >> 1;                       // group of 8 samples (base tiles)
        const int r0 = (warp & 1) * 4;                  // first of this warp's 4 rows in the group
        uint32_t it = 0, n_drained = 0;
        bool ok = true;
        bool pend = false, pend_first = false;
        int pend_sp = 0, pend_ot = 0, pend_ct = 0;
        auto drain = [&]() -> bool {
            // Partial sums live in a blocked layout so that a warp (32 consecutive rows) touches
            // contiguous memory: tile (split, o-tile, c-tile) -> [half][column / 4][row][4 floats].
            float4* tile = reinterpret_cast<float4*>(partial) +
                           (((size_t)pend_sp * plan.n_otiles + pend_ot) * n_ctiles + pend_ct) * (size_t)(2 * 64 * 128);
            const int row = quad * 32 + lane;
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                if (!mbar_wait(smem_u32(&ctrl->chunkFull[h]), n_drained & 1u, abort_flag)) return false;
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = part; c < BLOCK_N / 32; c += 4) {
                    float4* dst = tile + ((size_t)h * 64 + c * 8) * 128 + row;
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + h * BLOCK_N + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (pend_first)
                            dst[(size_t)q * 128] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                               __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                        else
                            red_add_v4(reinterpret_cast<float*>(dst + (size_t)q * 128), __uint_as_float(r[4 * q]),
                                       __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                       __uint_as_float(r[4 * q + 3]));
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&ctrl->drained[h]));
            }
            ++n_drained;
            pend = false;
            return true;
        };

        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int sp, ot, ct;
            decode(item, sp, ot, ct);
            const bool spline = ct < plan.ct_spline;
            const int f_tile0 = spline ? 0 : (ct - plan.ct_spline) * 256;
            int64_t kb0, kb1;
            k_range(sp, kb0, kb1);
            // spline tiles: chunk g = 32 ct + 4 fq + q belongs to feature g / cpf and holds its slots
            // 8 (g % cpf) ..; the inputs of the next block of samples are loaded one iteration ahead
            int cf[4], ccw[4];
            {
                const int g0 = ct * 32 + fq * 4;
                const int cpf = WIDE ? ti.cpf : 1;
                cf[0] = g0 / cpf;
                ccw[0] = g0 - cf[0] * cpf;
#pragma unroll
                for (int q = 1; q < 4; ++q) {
                    cf[q] = cf[q - 1];
                    ccw[q] = ccw[q - 1] + 1;
                    if (ccw[q] == cpf) { cf[q] += 1; ccw[q] = 0; }
                }
            }
            const int f_sp = cf[0];
            float nx[4] = {0.f, 0.f, 0.f, 0.f};
            auto prefetch_spline = [&](int64_t kb) {
                const int64_t n = kb * BLOCK_K + n_loc;
#pragma unroll
                for (int q = 0; q < 4; ++q) nx[q] = 0.f;
                if (n < N && f_sp < I) {
                    const float* xr = x + (size_t)n * I;
                    if (!WIDE && vec_ok && f_sp + 4 <= I) {
                        const float4 v = __ldg(reinterpret_cast<const float4*>(xr + f_sp));
                        nx[0] = v.x; nx[1] = v.y; nx[2] = v.z; nx[3] = v.w;
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (cf[q] < I) nx[q] = (q > 0 && cf[q] == cf[q - 1]) ? nx[q - 1] : __ldg(xr + cf[q]);
                    }
                }
            };
            if (spline) prefetch_spline(kb0);
            // position inside the chain, kept as a counter: a 64-bit division per block in each of the 512
            // workers is a measurable share of their instruction stream
            int in_chain = 0;
            for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t stage = it % BWD_G_STAGES;
                const uint32_t g_hi = sbase + BWD_SMEM_G + stage * BWD_G_STAGE_BYTES;
                const uint32_t g_lo = g_hi + TILE_B_BYTES;
                const bool chunk_start = in_chain == 0;
                if (spline) {
                    float xv[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) xv[q] = nx[q];
                    if (kb + 1 < kb1) prefetch_spline(kb + 1);
                    const bool n_ok = kb * BLOCK_K + n_loc < N;
                    if (!mbar_wait(smem_u32(&ctrl->emptyG[stage]), ((it / BWD_G_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    // row = sample (k index), 128 B = 64 columns = 8 chunks of 8 slots
                    const int kk = n_loc & 7;
                    Window w;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int f = cf[q];
                        if (!WIDE || q == 0 || f != cf[q - 1]) {    // uniform over the warp
                            if (shared_grid)
                                w = eval_window<SPLIT, true, WIDE>(stab, ti, xv[q]);
                            else
                                w = eval_window<SPLIT, false, WIDE>(tab + (size_t)(f < I ? f : I - 1) * ti.fs, ti,
                                                                    xv[q]);
                        }
                        uint4 hi, lo;
                        place_window<SPLIT>(w, ccw[q], hi, lo);
                        if (!(n_ok && f < I)) {
                            hi = make_uint4(0, 0, 0, 0);
                            lo = hi;
                        }
                        const int fl = fq * 4 + q;                       // chunk within the tile, 0..31
                        const uint32_t off = (uint32_t)((fl >> 3) * 8 + (n_loc >> 3)) * 1024u + (uint32_t)kk * 128u +
                                             (uint32_t)(((fl & 7) ^ kk) << 4);
                        st_shared_v4(g_hi + off, hi);
                        if (SPLIT) st_shared_v4(g_lo + off, lo);
                    }
                } else {
                    // lane = chunk of 8 base features; columns c = 8*lane .. 8*lane+7
                    const int64_t nrow0 = kb * BLOCK_K + kg * 8 + r0;
                    const uint32_t atom = (uint32_t)((lane >> 3) * 8 + kg) * 1024u;   // [col group][sample group]
                    const int f0 = f_tile0 + lane * 8;
                    float xv[4][8];
#pragma unroll
                    for (int q = 0; q < 4; ++q) load_x8(x, nrow0 + q, nrow0 + q < N, I, f0, vec_ok != 0, xv[q]);
                    if (!mbar_wait(smem_u32(&ctrl->emptyG[stage]), ((it / BWD_G_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 hi, lo;
                        silu_chunk<SPLIT>(xv[q], hi, lo);
                        const int rr = r0 + q;
                        const uint32_t off = atom + (uint32_t)rr * 128u + (uint32_t)(((lane & 7) ^ rr) << 4);
                        st_shared_v4(g_hi + off, hi);
                        if (SPLIT) st_shared_v4(g_lo + off, lo);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullG[stage]));
                if (pend && chunk_start) {
                    if (!drain()) {
                        ok = false;
                        break;
                    }
                }
                if (++in_chain == plan.chunk_kb) in_chain = 0;
                if (in_chain == 0 || kb + 1 == kb1) {
                    pend = true;
                    pend_first = (kb - kb0) < plan.chunk_kb;
                    pend_sp = sp;
                    pend_ot = ot;
                    pend_ct = ct;
                }
            }
        }
        if (ok && pend) drain();
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, true, true);
            constexpr uint64_t dbase = make_sdesc_sw128(8192, 1024);
            uint32_t it = 0, dslot = 0, n_chunks = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int sp, ot, ct;
                decode(item, sp, ot, ct);
                int64_t kb0, kb1;
                k_range(sp, kb0, kb1);
                int in_chain = 0;
                for (int64_t kb = kb0; kb < kb1 && ok; ++kb, ++it) {
                    const uint32_t stage = it % BWD_G_STAGES;
                    const uint32_t g_hi = sbase + BWD_SMEM_G + stage * BWD_G_STAGE_BYTES;
                    const uint32_t g_lo = g_hi + TILE_B_BYTES;
                    const bool chunk_start = in_chain == 0;
                    if (++in_chain == plan.chunk_kb) in_chain = 0;
                    const bool chunk_end = in_chain == 0 || kb + 1 == kb1;
                    if (!mbar_wait(smem_u32(&ctrl->fullG[stage]), (it / BWD_G_STAGES) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    for (int h = 0; h < 2; ++h, ++dslot) {
                        if (chunk_start && n_chunks > 0) {
                            // half h may be overwritten only after the workers have drained it
                            if (!mbar_wait(smem_u32(&ctrl->drained[h]), (n_chunks - 1) & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                        }
                        const uint32_t slot = dslot % BWD_D_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->fullD[slot]), (dslot / BWD_D_SLOTS) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t d_hi = sbase + BWD_SMEM_D + slot * BWD_D_SLOT_BYTES;
                        const uint32_t d_lo = d_hi + TILE_A_BYTES;
                        const uint32_t d_tmem = tmem_base + h * BLOCK_N;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, d_hi + ks * 2048), sdesc_at(dbase, g_hi + ks * 2048),
                                       idesc, (!chunk_start || ks > 0) ? 1u : 0u);
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
                        // the half's chain is complete: its drain overlaps the MMAs of the other half
                        if (chunk_end) mma_commit(smem_u32(&ctrl->chunkFull[h]));
                    }
                    if (!ok) break;
                    mma_commit(smem_u32(&ctrl->emptyG[stage]));
                    if (chunk_end) ++n_chunks;
                }
            }
        }
    } else {
        if (lane == 0) {
            uint32_t dslot = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int sp, ot, ct;
                decode(item, sp, ot, ct);
                int64_t kb0, kb1;
                k_range(sp, kb0, kb1);
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
        if (lane == 0) report_status(status, kStatusTimeout);
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

// ---------------------------------------------------------------------------
// Input-gradient kernel:
//   DW[n, c] = sum_o dY[n, o] W[o, c]                       (tensor cores, K = outputs)
//   gx[n, f] = sum_j DW[n, 8 f + s + j] dB_j/dx(x[n,f]) + DW[n, CS + f] silu'(x[n,f])
// ---------------------------------------------------------------------------
// Both operands already exist as images: the dY image of the parameter-gradient kernel read as a
// K-major A operand (rows = samples, 128 B = 64 outputs) and the forward's weight image read as an
// MN-major B operand (rows = outputs, 128 B = 64 columns), so nothing is generated here: the 16
// worker warps only run the epilogue, which contracts every group of 8 accumulator columns with
// the derivative of the basis.  Work item = (128 samples, 256 features): one sub-tile of 256 base
// columns (stores gx) followed by eight sub-tiles of 32 features x 8 slots (add to gx); the two
// 256-column accumulators in TMEM alternate between consecutive sub-tiles.
constexpr int DX_A_STAGES = 2, DX_B_SLOTS = 5;
constexpr uint32_t DX_A_STAGE_BYTES = 2 * TILE_A_BYTES;                  // hi + lo, 128 n x 64 o
constexpr uint32_t DX_SMEM_A = 0;
constexpr uint32_t DX_SMEM_B = DX_SMEM_A + DX_A_STAGES * DX_A_STAGE_BYTES;
constexpr uint32_t DX_SMEM_CTRL = DX_SMEM_B + DX_B_SLOTS * TILE_B_BYTES;
constexpr uint32_t DX_CTRL_BYTES = 256 + TAB_SMEM_FLOATS * 4;
constexpr uint32_t DX_SMEM_BYTES = DX_SMEM_CTRL + DX_CTRL_BYTES;
static_assert(DX_SMEM_BYTES <= 232448, "input-gradient kernel shared memory exceeds 227 KB");

struct DxCtrl {
    uint64_t fullA[DX_A_STAGES], emptyA[DX_A_STAGES];
    uint64_t fullB[DX_B_SLOTS], emptyB[DX_B_SLOTS];
    uint64_t accFull[2], accEmpty[2];
    uint64_t epiDone;      // workers: the previous sub-tile's gx stores are visible
    uint64_t phaseDone;    // workers: the even chunks of a wide sub-tile have been added to gx
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(DxCtrl) <= 256, "control block too large");

struct DxParams {
    int64_t N;
    int I, O;
    int kb_spline, kb_total;       // column blocks of the forward weight image
    int n_otiles;                  // 256-output tiles of the weight image
    int n_ohalves;                 // 128-output groups of the dY image
    int64_t n_blocks64;            // 64-sample blocks of the dY image
    int kb_o;                      // 64-output k-blocks
    int kb_o_chunk;                // k-blocks accumulated in TMEM before the epilogue adds them to gx
    int n_fgroups;                 // groups of 256 features
    int has_base;
    int64_t n_items;
    int vec_ok;
    TabInfo ti;
};

template <int NTERMS, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_bwd_input_kernel(const float* __restrict__ x, const float* __restrict__ tab, const uint8_t* __restrict__ dyimg,
                    const uint8_t* __restrict__ wimg, float* __restrict__ gx, int* __restrict__ status,
                    const DxParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    DxCtrl* ctrl = reinterpret_cast<DxCtrl*>(smem + DX_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + DX_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool shared_grid = grid_is_shared(tab, P.I, P.ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < P.ti.fs) stab[threadIdx.x] = tab[threadIdx.x];

    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) report_status(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < DX_A_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullA[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyA[s]), 1);
        }
        for (int s = 0; s < DX_B_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullB[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyB[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctrl->accFull[s]), 1);
            mbar_init(smem_u32(&ctrl->accEmpty[s]), WORKER_THREADS);
        }
        mbar_init(smem_u32(&ctrl->epiDone), WORKER_THREADS);
        mbar_init(smem_u32(&ctrl->phaseDone), WORKER_THREADS);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    // A group of 256 features owns 256 cpf chunks = 8 cpf spline sub-tiles of 32 chunks.
    const int cpf = WIDE ? P.ti.cpf : 1;
    const int sub_spline = 8 * cpf;
    const int n_sub = sub_spline + (P.has_base ? 1 : 0);    // sub-tiles per item
    // The reduction over the outputs is cut into chunks of kb_o_chunk k-blocks: an item runs its
    // sub-tiles once per chunk, and every pass after the first adds to gx.
    const int n_oc = (P.kb_o + P.kb_o_chunk - 1) / P.kb_o_chunk;
    // sub-tile j of feature group fg -> first column block of the weight image, and whether it is
    // the base sub-tile
    auto sub_info = [&](int fg, int j, bool& is_base, int& cb0) {
        is_base = P.has_base && j == 0;
        const int t = P.has_base ? j - 1 : j;               // spline sub-tile index
        cb0 = is_base ? P.kb_spline + fg * 4 : (fg * sub_spline + t) * 4;
    };

    if (warp < WORKER_WARPS) {
        // ===== workers: epilogue only =====
        const int quad = warp & 3, part = warp >> 2;
        const int row = quad * 32 + lane;
        uint32_t sub = 0;                                   // running sub-tile counter
        uint32_t n_phase = 0;                               // completed phase barriers (wide grids)
        for (int64_t item = blockIdx.x; item < P.n_items; item += gridDim.x) {
            const int64_t mt = item / P.n_fgroups;
            const int fg = (int)(item - mt * P.n_fgroups);
            const int64_t n = mt * BLOCK_M + row;
            const bool row_ok = n < P.N;
            const float* xrow = x + (size_t)(row_ok ? n : 0) * P.I;
            float* grow = gx + (size_t)(row_ok ? n : 0) * P.I;
            bool ok = true;
            for (int pass = 0; pass < n_oc * n_sub; ++pass, ++sub) {
                const int oc = pass / n_sub, j = pass - oc * n_sub;
                bool is_base;
                int cb0;
                sub_info(fg, j, is_base, cb0);
                const uint32_t buf = sub & 1u;
                if (!mbar_wait(smem_u32(&ctrl->accFull[buf]), (sub >> 1) & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                // gx of this item was (partly) written by other threads in the previous sub-tile
                if (sub > 0 && !mbar_wait(smem_u32(&ctrl->epiDone), (sub - 1) & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                if (WIDE && !is_base) {
                    // A feature's chunks are spread over column groups (other threads) and sub-tiles,
                    // but the window of one input touches at most two neighbouring chunks of its
                    // feature.  Chunks with an even index within their feature are added to gx
                    // first, the odd ones after a barrier: in each phase an element of gx has at
                    // most one writer, so the sums do not depend on scheduling.
                    const int t = P.has_base ? j - 1 : j;
                    const int gbase = (fg * sub_spline + t) * 32;           // first chunk of the sub-tile
#pragma unroll 1
                    for (int phase = 0; phase < 2 && ok; ++phase) {
                        if (phase == 1) {
                            mbar_arrive(smem_u32(&ctrl->phaseDone));
                            if (!mbar_wait(smem_u32(&ctrl->phaseDone), n_phase & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            ++n_phase;
                        }
#pragma unroll 1
                        for (int c = part; c < BLOCK_N / 32; c += 4) {
                            const int g0 = gbase + c * 4;
                            int f = g0 / cpf;
                            int cw = g0 - f * cpf;
                            if (f >= P.I) continue;                         // uniform over the warp
                            uint32_t r[32];
                            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BLOCK_N + c * 32, r);
                            tmem_ld_wait();
                            if (!row_ok) continue;
                            int fprev = -1, s = 0;
                            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                if (f < P.I && (cw & 1) == phase) {
                                    if (f != fprev) {
                                        s = eval_feature_deriv<false, true>(tab + (size_t)f * P.ti.fs, P.ti,
                                                                            __ldg(xrow + f), d);
                                        fprev = f;
                                    }
                                    const int sp = s - 8 * cw;              // window start within this chunk
                                    if (sp > -4 && sp < 8) {
                                        float acc = 0.f;
#pragma unroll
                                        for (int slot = 0; slot < 8; ++slot) {
                                            const int jj = slot - sp;
                                            float dv = 0.f;
#pragma unroll
                                            for (int w = 0; w < 4; ++w) dv = (jj == w) ? d[w] : dv;
                                            acc = fmaf(__uint_as_float(r[8 * e + slot]), dv, acc);
                                        }
                                        grow[f] += acc;
                                    }
                                }
                                if (++cw == cpf) {
                                    cw = 0;
                                    ++f;
                                }
                            }
                        }
                    }
                    if (!ok) break;
                } else {
#pragma unroll 1
                for (int c = part; c < BLOCK_N / 32; c += 4) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BLOCK_N + c * 32, r);
                    tmem_ld_wait();
                    if (!row_ok) continue;
                    if (is_base) {
                        const int f0 = fg * 256 + c * 32;           // 32 features
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const int f = f0 + 4 * q;
                            if (f >= P.I) break;
                            float xv[4] = {0.f, 0.f, 0.f, 0.f};
                            if (P.vec_ok && f + 4 <= P.I) {
                                const float4 v = __ldg(reinterpret_cast<const float4*>(xrow + f));
                                xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                            } else {
                                for (int e = 0; e < 4; ++e)
                                    if (f + e < P.I) xv[e] = __ldg(xrow + f + e);
                            }
                            float o[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) o[e] = __uint_as_float(r[4 * q + e]) * silu_grad_fast(xv[e]);
                            if (P.vec_ok && f + 4 <= P.I) {
                                float4* dst = reinterpret_cast<float4*>(grow + f);
                                if (oc > 0) {
                                    const float4 old = *dst;
                                    o[0] += old.x; o[1] += old.y; o[2] += old.z; o[3] += old.w;
                                }
                                *dst = make_float4(o[0], o[1], o[2], o[3]);
                            } else {
                                for (int e = 0; e < 4; ++e)
                                    if (f + e < P.I) grow[f + e] = oc > 0 ? grow[f + e] + o[e] : o[e];
                            }
                        }
                    } else {
                        const int t = P.has_base ? j - 1 : j;
                        const int f0 = fg * 256 + t * 32 + c * 4;   // 4 features x 8 slots
                        if (f0 >= P.I) continue;
                        float xv[4] = {0.f, 0.f, 0.f, 0.f};
                        if (P.vec_ok && f0 + 4 <= P.I) {
                            const float4 v = __ldg(reinterpret_cast<const float4*>(xrow + f0));
                            xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                        } else {
                            for (int e = 0; e < 4; ++e)
                                if (f0 + e < P.I) xv[e] = __ldg(xrow + f0 + e);
                        }
                        float o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int f = f0 + e;
                            float d[4];
                            int s;
                            if (shared_grid)
                                s = eval_feature_deriv<true, false>(stab, P.ti, xv[e], d);
                            else
                                s = eval_feature_deriv<false, false>(tab + (size_t)(f < P.I ? f : P.I - 1) * P.ti.fs, P.ti,
                                                              xv[e], d);
                            float acc = 0.f;
#pragma unroll
                            for (int slot = 0; slot < 8; ++slot) {
                                const int jj = slot - s;               // window index of this slot
                                float dv = 0.f;
#pragma unroll
                                for (int w = 0; w < 4; ++w) dv = (jj == w) ? d[w] : dv;
                                acc = fmaf(__uint_as_float(r[8 * e + slot]), dv, acc);
                            }
                            o[e] = acc;
                        }
                        if (P.vec_ok && f0 + 4 <= P.I) {
                            float4* dst = reinterpret_cast<float4*>(grow + f0);
                            if (P.has_base || oc > 0) {
                                const float4 old = *dst;
                                o[0] += old.x; o[1] += old.y; o[2] += old.z; o[3] += old.w;
                            }
                            *dst = make_float4(o[0], o[1], o[2], o[3]);
                        } else {
                            for (int e = 0; e < 4; ++e)
                                if (f0 + e < P.I) grow[f0 + e] = (P.has_base || oc > 0) ? grow[f0 + e] + o[e] : o[e];
                        }
                    }
                }
                }
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&ctrl->accEmpty[buf]));
                mbar_arrive(smem_u32(&ctrl->epiDone));
            }
            if (!ok) break;
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, false, true);       // A K-major, B MN-major
            constexpr uint64_t da = make_sdesc_sw128(16, 1024);
            constexpr uint64_t db = make_sdesc_sw128(8192, 1024);
            uint32_t it = 0, bslot = 0, sub = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
                for (int pass = 0; pass < n_oc * n_sub && ok; ++pass, ++sub) {
                    const int oc = pass / n_sub;
                    const int ko0 = oc * P.kb_o_chunk, ko1 = (ko0 + P.kb_o_chunk < P.kb_o) ? ko0 + P.kb_o_chunk : P.kb_o;
                    const uint32_t buf = sub & 1u;
                    if (!mbar_wait(smem_u32(&ctrl->accEmpty[buf]), ((sub >> 1) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
                    for (int ko = ko0; ko < ko1; ++ko, ++it) {
                        const uint32_t stage = it % DX_A_STAGES;
                        const uint32_t a_hi = sbase + DX_SMEM_A + stage * DX_A_STAGE_BYTES;
                        const uint32_t a_lo = a_hi + TILE_A_BYTES;
                        const uint32_t slot_h = bslot % DX_B_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->fullA[stage]), (it / DX_A_STAGES) & 1u, abort_flag) ||
                            !mbar_wait(smem_u32(&ctrl->fullB[slot_h]), (bslot / DX_B_SLOTS) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t b_hi = sbase + DX_SMEM_B + slot_h * TILE_B_BYTES;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(da, a_hi + ks * 32), sdesc_at(db, b_hi + ks * 2048), idesc,
                                       (ko > ko0 || ks > 0) ? 1u : 0u);
                        if (SPLIT) {
#pragma unroll
                            for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                                mma_f16_ss(d_tmem, sdesc_at(da, a_lo + ks * 32), sdesc_at(db, b_hi + ks * 2048),
                                           idesc, 1u);
                        }
                        mma_commit(smem_u32(&ctrl->emptyB[slot_h]));
                        ++bslot;
                        if (SPLIT) {
                            const uint32_t slot_l = bslot % DX_B_SLOTS;
                            if (!mbar_wait(smem_u32(&ctrl->fullB[slot_l]), (bslot / DX_B_SLOTS) & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t b_lo = sbase + DX_SMEM_B + slot_l * TILE_B_BYTES;
#pragma unroll
                            for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                                mma_f16_ss(d_tmem, sdesc_at(da, a_hi + ks * 32), sdesc_at(db, b_lo + ks * 2048),
                                           idesc, 1u);
                            mma_commit(smem_u32(&ctrl->emptyB[slot_l]));
                            ++bslot;
                        }
                        mma_commit(smem_u32(&ctrl->emptyA[stage]));
                    }
                    if (ok) mma_commit(smem_u32(&ctrl->accFull[buf]));
                }
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk copies: dY tiles (A) and weight tiles (B) =====
            uint32_t it = 0, bslot = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
                const int64_t mt = item / P.n_fgroups;
                const int fg = (int)(item - mt * P.n_fgroups);
                for (int pass = 0; pass < n_oc * n_sub && ok; ++pass) {
                    const int oc = pass / n_sub, j = pass - oc * n_sub;
                    const int ko0 = oc * P.kb_o_chunk, ko1 = (ko0 + P.kb_o_chunk < P.kb_o) ? ko0 + P.kb_o_chunk : P.kb_o;
                    bool is_base;
                    int cb0;
                    sub_info(fg, j, is_base, cb0);
                    for (int ko = ko0; ko < ko1 && ok; ++ko, ++it) {
                        // A: 128 samples x 64 outputs = two 64-sample blocks of the dY image
                        const uint32_t stage = it % DX_A_STAGES;
                        if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / DX_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        {
                            const uint32_t bar = smem_u32(&ctrl->fullA[stage]);
                            const int terms = SPLIT ? 2 : 1;
                            // the second 64-sample block may lie beyond the batch: its rows are then
                            // left as they are (they only feed accumulator rows that are never stored)
                            const int halves = (mt * 2 + 1 < P.n_blocks64) ? 2 : 1;
                            mbar_arrive_expect_tx(bar, (uint32_t)(terms * halves) * 8192u);
                            const int oh = ko >> 1, og = ko & 1;
                            for (int term = 0; term < terms; ++term)
                                for (int hn = 0; hn < halves; ++hn) {
                                    const int64_t nb = mt * 2 + hn;
                                    const uint8_t* src = dyimg + (((size_t)nb * P.n_ohalves + oh) * 2 + term) * TILE_A_BYTES +
                                                         (size_t)og * 8192;
                                    bulk_g2s(sbase + DX_SMEM_A + stage * DX_A_STAGE_BYTES + term * TILE_A_BYTES + hn * 8192,
                                             src, 8192, bar);
                                }
                        }
                        // B: 256 columns x 64 outputs = four column blocks of the weight image
                        const int ot = ko >> 2, og8 = ko & 3;
                        int n_cb = P.kb_total - cb0;
                        if (is_base) {
                            const int left = P.kb_total - cb0;
                            n_cb = left < 4 ? left : 4;
                        } else {
                            const int left = P.kb_spline - cb0;
                            n_cb = left < 4 ? left : 4;
                        }
                        if (n_cb < 0) n_cb = 0;
                        for (int term = 0; term < (SPLIT ? 2 : 1); ++term, ++bslot) {
                            const uint32_t slot = bslot % DX_B_SLOTS;
                            if (!mbar_wait(smem_u32(&ctrl->emptyB[slot]), ((bslot / DX_B_SLOTS) & 1u) ^ 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            const uint32_t bar = smem_u32(&ctrl->fullB[slot]);
                            if (n_cb == 0) {
                                mbar_arrive(bar);
                            } else {
                                mbar_arrive_expect_tx(bar, (uint32_t)n_cb * 8192u);
                                for (int cg = 0; cg < n_cb; ++cg) {
                                    const uint8_t* src = wimg + (((size_t)ot * P.kb_total + cb0 + cg) * 2 + term) * TILE_B_BYTES +
                                                         (size_t)og8 * 8192;
                                    bulk_g2s(sbase + DX_SMEM_B + slot * TILE_B_BYTES + cg * 8192, src, 8192, bar);
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    if (*abort_flag) {
        if (lane == 0) report_status(status, kStatusTimeout);
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

// Sums the per-split slabs (blocked layout of the drain) and applies the scaler algebra:
// gsw = scaler * D, gscaler = sum_r sw * D, gbw = base column.  A block handles 32 outputs x 8
// features: the slabs are read with the output index fastest (contiguous 16-byte pieces per warp),
// transposed through shared memory, and the parameter-shaped tensors are then read / written with
// the feature index fastest (256 contiguous bytes per output row).
constexpr int FIN_TO = 32, FIN_TI = 8;
__global__ void __launch_bounds__(FIN_TO * FIN_TI)
finalize_blocked_kernel(const float* __restrict__ partial, BwdPlan plan,
                        const float* __restrict__ sw, const float* __restrict__ scaler,
                        float* __restrict__ gsw, float* __restrict__ gscaler,
                        float* __restrict__ gbw, int O, int I, int R) {
    __shared__ float Ds[FIN_TO][FIN_TI * 8 + 1];
    __shared__ float Bs[FIN_TO][FIN_TI + 1];
    const int o0 = blockIdx.x * FIN_TO, i0 = blockIdx.y * FIN_TI;
    const int n_ctiles = plan.n_ctiles();
    {
        const int ol = threadIdx.x & (FIN_TO - 1), il = threadIdx.x / FIN_TO;
        const int o = o0 + ol, i = i0 + il;
        float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float db = 0.f;
        if (o < O && i < I) {
            const int ot = o >> 8, h = (o >> 7) & 1, row = o & 127;
            auto tile_ptr = [&](int sp, int ct) -> const float4* {
                return reinterpret_cast<const float4*>(partial) +
                       ((((size_t)sp * plan.n_otiles + ot) * n_ctiles + ct) * 2 + h) * (size_t)(64 * 128) + row;
            };
            if (gsw || gscaler) {
                const int ct = i >> 5, fl = i & 31;
                for (int sp = 0; sp < plan.splits; ++sp) {
                    const float4* t = tile_ptr(sp, ct);
                    const float4 a = t[(size_t)(fl * 2) * 128], b = t[(size_t)(fl * 2 + 1) * 128];
                    d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w;
                    d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
                }
            }
            if (gbw) {
                const int ct = plan.ct_spline + (i >> 8), c = i & 255;
                for (int sp = 0; sp < plan.splits; ++sp) {
                    const float4 a = tile_ptr(sp, ct)[(size_t)(c >> 2) * 128];
                    db += (c & 3) == 0 ? a.x : ((c & 3) == 1 ? a.y : ((c & 3) == 2 ? a.z : a.w));
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) Ds[ol][il * 8 + r] = d[r];
        Bs[ol][il] = db;
    }
    __syncthreads();
    {
        const int il = threadIdx.x & (FIN_TI - 1), ol = threadIdx.x / FIN_TI;
        const int o = o0 + ol, i = i0 + il;
        if (o >= O || i >= I) return;
        const size_t oi = (size_t)o * I + i;
        if (gsw || gscaler) {
            const float sc = scaler ? scaler[oi] : 1.0f;
            float gs = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < R) {
                    const float d = Ds[ol][il * 8 + r];
                    if (gsw) gsw[oi * R + r] = scaler ? sc * d : d;
                    if (gscaler) gs += sw[oi * R + r] * d;
                }
            }
            if (gscaler) gscaler[oi] = gs;
        }
        if (gbw) gbw[oi] = Bs[ol][il];
    }
}

// The same reduction for features that own more than one chunk of 8 slots (R > 8): one thread
// per (output, feature) with the output index fastest, so that the slabs are read in contiguous
// 16-byte pieces per warp.
__global__ void __launch_bounds__(256)
finalize_wide_kernel(const float* __restrict__ partial, BwdPlan plan, int cpf,
                     const float* __restrict__ sw, const float* __restrict__ scaler,
                     float* __restrict__ gsw, float* __restrict__ gscaler,
                     float* __restrict__ gbw, int O, int I, int R) {
    const int n_ctiles = plan.n_ctiles();
    const int64_t total = (int64_t)O * I;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int o = (int)(idx % O), i = (int)(idx / O);
        const int ot = o >> 8, h = (o >> 7) & 1, row = o & 127;
        auto tile_ptr = [&](int sp, int ct) -> const float4* {
            return reinterpret_cast<const float4*>(partial) +
                   ((((size_t)sp * plan.n_otiles + ot) * n_ctiles + ct) * 2 + h) * (size_t)(64 * 128) + row;
        };
        const size_t oi = (size_t)o * I + i;
        if (gsw || gscaler) {
            const float sc = scaler ? scaler[oi] : 1.0f;
            float gs = 0.f;
            for (int cw = 0; cw < cpf; ++cw) {
                const int g = i * cpf + cw, ct = g >> 5, gl = g & 31;
                float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int sp = 0; sp < plan.splits; ++sp) {
                    const float4* t = tile_ptr(sp, ct);
                    const float4 a = t[(size_t)(gl * 2) * 128], b = t[(size_t)(gl * 2 + 1) * 128];
                    d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w;
                    d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int r = cw * 8 + e;
                    if (r < R) {
                        if (gsw) gsw[oi * R + r] = scaler ? sc * d[e] : d[e];
                        if (gscaler) gs += sw[oi * R + r] * d[e];
                    }
                }
            }
            if (gscaler) gscaler[oi] = gs;
        }
        if (gbw) {
            const int ct = plan.ct_spline + (i >> 8), c = i & 255;
            float db = 0.f;
            for (int sp = 0; sp < plan.splits; ++sp) {
                const float4 a = tile_ptr(sp, ct)[(size_t)(c >> 2) * 128];
                db += (c & 3) == 0 ? a.x : ((c & 3) == 1 ? a.y : ((c & 3) == 2 ? a.z : a.w));
            }
            gbw[oi] = db;
        }
    }
}

// Chunk lengths (k-blocks accumulated in TMEM between drains).  Every tensor-core accumulation
// truncates toward zero, i.e. shrinks the running sum by a fraction of an ulp; over a chain the
// error grows like (number of accumulations) x |partial sums| and is systematic.  A drain adds the
// chain's result to the running total in float32 with round-to-nearest (in L2, red.global.add) and
// restarts the chain at zero.  Measured against float64 (max-norm relative), 12 accumulations per
// block of 64:
//   forward, spline-dominated weights, 1024 features (144 blocks): one chain 3.2e-5; the error is
//     proportional to the chain length, chains of 24 blocks stay at the operand-split floor
//     (5e-6 .. 7e-6).  (With the reference's initialisation the base branch dominates y and even
//     one chain of 144 blocks measures 5.4e-6, which is why only general weights show it.)
//     4096 features: chains of 144 / 48 / 36 / 24 blocks give 1.55e-5 / 9.8e-6 / 8.5e-6 / 5.4e-6;
//   parameter gradients, 65536 samples: chains of 16 / 32 / 64 blocks of 64 samples give 5.4e-6 /
//     8.4e-6 / 1.4e-5;
//   input gradient, 4096 outputs (64 blocks): one chain 1.5e-5, chains of 32 / 24 / 16 / 8 blocks
//     8.5e-6 / 6.3e-6 / 6.7e-6 / 4.7e-6 (1024 outputs, 16 blocks: 5.9e-6, unaffected).
// They are part of the numerical contract; kanb200_set_accumulation_chunks can only shorten them.
constexpr int kFwdChunkKb = 24;       // forward: 64-column blocks per chain
constexpr int kBwdChunkKb = 16;       // parameter gradients: 64-sample blocks per chain
constexpr int kDxChunkKb = 24;        // input gradient: 64-output blocks per chain
int g_fwd_chunk = kFwdChunkKb, g_bwd_chunk = kBwdChunkKb, g_dx_chunk = kDxChunkKb;
inline int fwd_chunk_kb(int) { return g_fwd_chunk; }
inline int bwd_chunk_kb() { return g_bwd_chunk; }
inline int dx_chunk_kb() { return g_dx_chunk; }

inline BwdPlan plan_bwd(const LayerShape& s, bool has_base) {
    BwdPlan p;
    p.n_otiles = (s.O + BLOCK_N - 1) / BLOCK_N;
    p.ct_spline = (s.I * make_tab_info(s.G, s.K).cpf + 31) / 32;
    p.ct_base = has_base ? (s.I + 255) / 256 : 0;
    p.kb_total = (s.N + BLOCK_K - 1) / BLOCK_K;
    p.chunk_kb = bwd_chunk_kb();
    const int64_t tiles = (int64_t)p.n_otiles * p.n_ctiles();
    int64_t splits = sm_count() / tiles;
    if (splits < 1) splits = 1;
    if (splits > p.kb_total) splits = p.kb_total;
    if (splits > 32) splits = 32;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    p.splits = (int)((p.kb_total + p.kb_per_split - 1) / p.kb_per_split);
    return p;
}

inline size_t table_bytes(const LayerShape& s) {
    return align256((size_t)s.I * make_tab_info(s.G, s.K).fs * sizeof(float));
}

inline cudaError_t launch_table(const float* grid, float* tab, const LayerShape& s, cudaStream_t st) {
    const TabInfo ti = make_tab_info(s.G, s.K);
    const int work = s.I * (ti.nk + 1);
    build_poly_table_kernel<<<(work + 127) / 128, 128, 0, st>>>(grid, tab, s.I, s.G, s.K, ti);
    return cudaGetLastError();
}

struct FwdLayout {
    ColumnSpace cs;
    int n_otiles;
    size_t wimg_bytes;
};
inline FwdLayout fwd_layout(const LayerShape& s, bool has_base) {
    FwdLayout L;
    L.cs = column_space(s.I, make_tab_info(s.G, s.K).cpf, has_base);
    L.n_otiles = (s.O + BLOCK_N - 1) / BLOCK_N;
    L.wimg_bytes = (size_t)L.n_otiles * L.cs.kb_total() * 2 * TILE_B_BYTES;
    return L;
}

// Number of separately stored chains the forward would split a tile into for this batch (1 = no
// split): a tile's chain over the columns is serial, so a batch of few row tiles leaves most SMs idle
// unless the chains of chunk_kb blocks -- which are drained separately anyway -- become work items.
inline int forward_ksplit(const LayerShape& s, bool has_base, int64_t n_tiles) {
    const int kb_total = fwd_layout(s, has_base).cs.kb_total();
    const int chains = (kb_total + fwd_chunk_kb(kb_total) - 1) / fwd_chunk_kb(kb_total);
    return (chains > 1 && n_tiles * 2 <= sm_count()) ? chains : 1;
}
// Bytes of the partial results for the most finely split case of this shape.
inline size_t forward_slab_bytes(const LayerShape& s, bool has_base) {
    const FwdLayout L = fwd_layout(s, has_base);
    const int64_t row_tiles = (s.N + BLOCK_M - 1) / BLOCK_M;
    const int k = forward_ksplit(s, has_base, row_tiles * ((L.n_otiles + 1) / 2));     // the smaller tile count
    return k > 1 ? align256((size_t)k * (size_t)s.N * s.O * sizeof(float)) : 0;
}

struct BwdLayout {
    BwdPlan plan;
    size_t dyimg_bytes, partial_bytes;
};
inline BwdLayout bwd_layout(const LayerShape& s, bool has_base) {
    BwdLayout L;
    L.plan = plan_bwd(s, has_base);
    L.dyimg_bytes = (size_t)L.plan.kb_total * L.plan.n_otiles * 2 * BWD_D_SLOT_BYTES;
    L.partial_bytes = (size_t)L.plan.splits * L.plan.slab_floats() * sizeof(float);
    return L;
}

}  // namespace

size_t tc_table_bytes(const LayerShape& s) { return table_bytes(s); }
int tc_table_stride(const LayerShape& s) { return make_tab_info(s.G, s.K).fs; }
cudaError_t tc_build_table(const float* grid, float* tab, const LayerShape& s, cudaStream_t st) {
    return launch_table(grid, tab, s, st);
}

// Shorter accumulation chains (never longer than the built-in lengths, so the stated tolerance
// always holds); 0 keeps a value.
// Which forward kernel runs: -1 = by shape, 0 = generated operand in shared memory, 1 = in tensor memory.
int g_fwd_variant = -1;
void tc_set_forward_variant(int v) { g_fwd_variant = v < 0 ? -1 : (v > 0 ? 1 : 0); }

void tc_set_chunks(int fwd_kb, int bwd_kb, int dx_kb) {
    auto clamp = [](int v, int cur, int max) { return v <= 0 ? cur : (v < 1 ? 1 : (v > max ? max : v)); };
    g_fwd_chunk = clamp(fwd_kb, g_fwd_chunk, kFwdChunkKb);
    g_bwd_chunk = clamp(bwd_kb, g_bwd_chunk, kBwdChunkKb);
    g_dx_chunk = clamp(dx_kb, g_dx_chunk, kDxChunkKb);
}

bool tc_supported(const LayerShape& s) {
    // any grid the layer accepts (G + 2 K <= 71); the window of k + 1 <= 4 values is what the
    // table entries hold
    return s.K >= 1 && s.K <= 3 && s.G >= 1 && s.T() <= 72 && s.N >= 1 && s.I >= 1 && s.O >= 1;
}

size_t tc_workspace(int op, const LayerShape& s, bool need_x, bool need_param) {
    // Sized for a layer with a base branch (the larger case).
    if (op == 0)
        return kWsHeader + table_bytes(s) + align256(fwd_layout(s, true).wimg_bytes) + forward_slab_bytes(s, true);
    size_t b = kWsHeader + table_bytes(s);
    BwdLayout L = bwd_layout(s, true);
    if (need_param || need_x) b += align256(L.dyimg_bytes);
    if (need_param) b += align256(L.partial_bytes);
    if (need_x) b += align256(fwd_layout(s, true).wimg_bytes);
    return b;
}

// y = slab[0] + slab[1] + ... in that order (the forward's per-chain partial results, small batches).
__global__ void sum_forward_slabs_kernel(const float* __restrict__ slab, float* __restrict__ y, int64_t count,
                                         int n_slabs, int vec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        const float4* s4 = reinterpret_cast<const float4*>(slab);
        float4* y4 = reinterpret_cast<float4*>(y);
        const int64_t c4 = count / 4;
        for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < c4; e += stride) {
            float4 a = s4[e];
            for (int c = 1; c < n_slabs; ++c) {
                const float4 b = s4[(size_t)c * c4 + e];
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            }
            y4[e] = a;
        }
    } else {
        for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += stride) {
            float a = slab[e];
            for (int c = 1; c < n_slabs; ++c) a += slab[(size_t)c * count + e];
            y[e] = a;
        }
    }
}

// Table of the knots and bf16 image of the effective weights: everything the forward kernels need
// besides x.  They depend on the parameters only, so inference with fixed parameters builds them once
// (tc_prepare_forward) and every later call runs the contraction alone (tc_forward_prepared).
namespace {
cudaError_t build_forward_operands(const float* grid, const float* bw, const float* sw, const float* scaler,
                                   float* tab, uint8_t* wimg, const LayerShape& s, cudaStream_t st) {
    const FwdLayout L = fwd_layout(s, bw != nullptr);
    const TabInfo ti = make_tab_info(s.G, s.K);
    const int kb_total = L.cs.kb_total();
    cudaError_t e0 = launch_table(grid, tab, s, st);
    if (e0 != cudaSuccess) return e0;
    const int64_t chunks = (int64_t)L.n_otiles * kb_total * BLOCK_N * 8;
    int blocks = (int)((chunks + 255) / 256);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    pack_weights_kernel<<<blocks, 256, 0, st>>>(sw, scaler, bw, wimg, s.O, s.I, s.R(), ti.cpf, L.cs.kb_spline,
                                                kb_total, L.n_otiles);
    return cudaGetLastError();
}
cudaError_t run_forward(int split_terms, const float* x, const float* tab, const uint8_t* wimg, float* y,
                        int* status, void* slab, size_t slab_bytes, const LayerShape& s, bool has_base,
                        cudaStream_t st);
}  // namespace

size_t tc_prepared_bytes(const LayerShape& s, bool has_base) {
    return table_bytes(s) + align256(fwd_layout(s, has_base).wimg_bytes);
}

cudaError_t tc_prepare_forward(const float* grid, const float* bw, const float* sw, const float* scaler,
                               const LayerShape& s, void* prepared, size_t prepared_bytes, cudaStream_t st) {
    if (!prepared || prepared_bytes < tc_prepared_bytes(s, bw != nullptr)) return cudaErrorMemoryAllocation;
    float* tab = reinterpret_cast<float*>(prepared);
    uint8_t* wimg = reinterpret_cast<uint8_t*>(prepared) + table_bytes(s);
    return build_forward_operands(grid, bw, sw, scaler, tab, wimg, s, st);
}

cudaError_t tc_forward_prepared(int split_terms, const float* x, const void* prepared, size_t prepared_bytes,
                                bool has_base, float* y, const LayerShape& s, void* ws, size_t ws_bytes,
                                cudaStream_t st) {
    if (s.N == 0) return cudaSuccess;
    if (!prepared || prepared_bytes < tc_prepared_bytes(s, has_base)) return cudaErrorMemoryAllocation;
    if (!ws || ws_bytes < kWsHeader) return cudaErrorMemoryAllocation;
    const float* tab = reinterpret_cast<const float*>(prepared);
    const uint8_t* wimg = reinterpret_cast<const uint8_t*>(prepared) + table_bytes(s);
    return run_forward(split_terms, x, tab, wimg, y, reinterpret_cast<int*>(ws),
                       reinterpret_cast<uint8_t*>(ws) + kWsHeader, ws_bytes - kWsHeader, s, has_base, st);
}

cudaError_t tc_forward(int split_terms, const float* x, const float* grid, const float* bw, const float* sw,
                       const float* scaler, float* y, const LayerShape& s,
                       void* ws, size_t ws_bytes, cudaStream_t st) {
    if (s.N == 0) return cudaSuccess;
    const bool has_base = bw != nullptr;
    FwdLayout L = fwd_layout(s, has_base);
    if (!ws || ws_bytes < kWsHeader + table_bytes(s) + L.wimg_bytes) return cudaErrorMemoryAllocation;
    int* status = reinterpret_cast<int*>(ws);
    float* tab = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + kWsHeader);
    uint8_t* wimg = reinterpret_cast<uint8_t*>(ws) + kWsHeader + table_bytes(s);
    cudaError_t e = build_forward_operands(grid, bw, sw, scaler, tab, wimg, s, st);
    if (e != cudaSuccess) return e;
    const size_t used = kWsHeader + table_bytes(s) + align256(L.wimg_bytes);
    return run_forward(split_terms, x, tab, wimg, y, status, reinterpret_cast<uint8_t*>(ws) + used,
                       ws_bytes > used ? ws_bytes - used : 0, s, has_base, st);
}

namespace {
cudaError_t run_forward(int split_terms, const float* x, const float* tab, const uint8_t* wimg, float* y,
                        int* status, void* slab, size_t slab_bytes, const LayerShape& s, bool has_base,
                        cudaStream_t st) {
    const FwdLayout L = fwd_layout(s, has_base);
    const TabInfo ti = make_tab_info(s.G, s.K);
    const int kb_total = L.cs.kb_total();
    FwdParams P;
    P.N = s.N; P.I = s.I; P.O = s.O; P.G = s.G;
    P.kb_spline = L.cs.kb_spline; P.kb_total = kb_total;
    P.n_otiles = L.n_otiles; P.n_opairs = (L.n_otiles + 1) / 2;
    P.n_tiles = ((s.N + BLOCK_M - 1) / BLOCK_M) * P.n_opairs;
    P.chunk_kb = fwd_chunk_kb(kb_total);
    P.vec_x = ((s.I & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    P.vec_x2 = ((s.I & 1) == 0) && ((reinterpret_cast<uintptr_t>(x) & 7) == 0);
    P.vec_y = ((s.O & 3) == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    P.ti = ti;
    cudaError_t e = cudaSuccess;
    // layers of up to 256 outputs (a single output tile) gain from the tensor-memory operand: the generated
    // tile serves one accumulator either way, and shared memory is left to the weight tiles
    const bool operand_in_tmem = g_fwd_variant < 0 ? P.n_otiles == 1 : g_fwd_variant == 1;
    if (operand_in_tmem) P.n_tiles = ((s.N + BLOCK_M - 1) / BLOCK_M) * P.n_otiles;      // one 256-output tile each
    // small batches: one work item per chain, partial results in the workspace (when it has the room)
    P.n_ksplit = forward_ksplit(s, has_base, P.n_tiles);
    if (P.n_ksplit > 1 && (!slab || slab_bytes < (size_t)P.n_ksplit * (size_t)s.N * s.O * sizeof(float))) P.n_ksplit = 1;
    P.slab = reinterpret_cast<float*>(slab);
    const int64_t n_items = P.n_items();
    const int blocks = (int)(n_items < sm_count() ? n_items : sm_count());
#define KAN_FWD(NT, W)                                                                                         \
    do {                                                                                                      \
        if (operand_in_tmem) {                                                                                \
            e = ensure_dynamic_smem<tc_forward_ts_kernel<NT, W>>((int)FTS_SMEM_BYTES);                        \
            if (e == cudaSuccess)                                                                             \
                tc_forward_ts_kernel<NT, W><<<blocks, TC_THREADS, FTS_SMEM_BYTES, st>>>(x, tab, wimg, y,      \
                                                                                         status, P);         \
            break;                                                                                            \
        }                                                                                                     \
        e = ensure_dynamic_smem<tc_forward_kernel<NT, W>>((int)FWD_SMEM_BYTES);                               \
        if (e == cudaSuccess)                                                                                 \
            tc_forward_kernel<NT, W><<<blocks, TC_THREADS, FWD_SMEM_BYTES, st>>>(x, tab, wimg, y, status, P); \
    } while (0)
    if (ti.cpf == 1) {
        if (split_terms == 3) KAN_FWD(3, false); else KAN_FWD(1, false);
    } else {
        if (split_terms == 3) KAN_FWD(3, true); else KAN_FWD(1, true);
    }
#undef KAN_FWD
    if (e != cudaSuccess) return e;
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (P.n_ksplit > 1) {
        const int64_t count = s.N * (int64_t)s.O;
        const int vec = (count % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
        const int64_t work = vec ? count / 4 : count;
        int rblocks = (int)((work + 255) / 256 < (int64_t)sm_count() * 8 ? (work + 255) / 256 : (int64_t)sm_count() * 8);
        sum_forward_slabs_kernel<<<rblocks, 256, 0, st>>>(P.slab, y, count, P.n_ksplit, vec);
        e = cudaGetLastError();
    }
    return e;
}
}  // namespace

cudaError_t tc_backward(int split_terms, const float* dY, int64_t ldy, const float* x, const float* grid,
                        const float* bw, const float* sw, const float* scaler, float* gx, float* gbw, float* gsw,
                        float* gscaler, const LayerShape& s, void* ws, size_t ws_bytes, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    const bool has_base = bw != nullptr;
    const bool need_param = gsw || gscaler || (gbw && has_base);
    if (s.N == 0) return simt_backward<float>(dY, x, grid, bw, sw, scaler, gx, gbw, gsw, gscaler, s, nullptr, 0, st);
    const TabInfo ti = make_tab_info(s.G, s.K);
    const bool need_x = gx != nullptr;
    if (!need_param && !need_x) return cudaSuccess;

    BwdLayout L = bwd_layout(s, has_base);
    FwdLayout F = fwd_layout(s, has_base);
    size_t need = kWsHeader + table_bytes(s) + align256(L.dyimg_bytes);
    if (need_param) need += align256(L.partial_bytes);
    if (need_x) need += F.wimg_bytes;
    if (!ws || ws_bytes < need) return cudaErrorMemoryAllocation;
    int* status = reinterpret_cast<int*>(ws);
    float* tab = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + kWsHeader);
    uint8_t* dyimg = reinterpret_cast<uint8_t*>(ws) + kWsHeader + table_bytes(s);
    uint8_t* cursor = dyimg + align256(L.dyimg_bytes);
    float* partial = reinterpret_cast<float*>(cursor);
    if (need_param) cursor += align256(L.partial_bytes);
    uint8_t* wimg = cursor;

    if ((e = launch_table(grid, tab, s, st)) != cudaSuccess) return e;
    {
        const int64_t chunks = L.plan.kb_total * L.plan.n_otiles * 2 * 64 * 16;
        int blocks = (int)((chunks + 255) / 256 < (int64_t)sm_count() * 16 ? (chunks + 255) / 256
                                                                            : (int64_t)sm_count() * 16);
        pack_grad_out_kernel<<<blocks, 256, 0, st>>>(dY, ldy, dyimg, s.N, s.O, L.plan.kb_total,
                                                     L.plan.n_otiles * 2);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    const int vec_ok = ((s.I & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (need_param) {
        const int64_t items = L.plan.n_items();
        const int blocks = (int)(items < sm_count() ? items : sm_count());
#define KAN_BWD(NT, W)                                                                                         \
    do {                                                                                                      \
        e = ensure_dynamic_smem<tc_bwd_param_kernel<NT, W>>((int)BWD_SMEM_BYTES);                             \
        if (e == cudaSuccess)                                                                                 \
            tc_bwd_param_kernel<NT, W><<<blocks, TC_THREADS, BWD_SMEM_BYTES, st>>>(                           \
                x, tab, dyimg, partial, status, s.N, s.I, s.O, L.plan, ti, vec_ok);                           \
    } while (0)
        if (ti.cpf == 1) {
            if (split_terms == 3) KAN_BWD(3, false); else KAN_BWD(1, false);
        } else {
            if (split_terms == 3) KAN_BWD(3, true); else KAN_BWD(1, true);
        }
#undef KAN_BWD
        if (e != cudaSuccess) return e;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        if (ti.cpf == 1) {
            dim3 fgrid((s.O + FIN_TO - 1) / FIN_TO, (s.I + FIN_TI - 1) / FIN_TI);
            finalize_blocked_kernel<<<fgrid, FIN_TO * FIN_TI, 0, st>>>(partial, L.plan, sw, scaler, gsw, gscaler,
                                                                       has_base ? gbw : nullptr, s.O, s.I, s.R());
        } else {
            const int64_t total = (int64_t)s.O * s.I;
            int fblocks = (int)((total + 255) / 256 < (int64_t)sm_count() * 16 ? (total + 255) / 256
                                                                               : (int64_t)sm_count() * 16);
            finalize_wide_kernel<<<fblocks, 256, 0, st>>>(partial, L.plan, ti.cpf, sw, scaler, gsw, gscaler,
                                                          has_base ? gbw : nullptr, s.O, s.I, s.R());
        }
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (need_x) {
        const int kb_total = F.cs.kb_total();
        {
            const int64_t chunks = (int64_t)F.n_otiles * kb_total * BLOCK_N * 8;
            int blocks = (int)((chunks + 255) / 256);
            if (blocks > sm_count() * 16) blocks = sm_count() * 16;
            pack_weights_kernel<<<blocks, 256, 0, st>>>(sw, scaler, bw, wimg, s.O, s.I, s.R(), ti.cpf, F.cs.kb_spline,
                                                        kb_total, F.n_otiles);
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        DxParams P;
        P.N = s.N; P.I = s.I; P.O = s.O;
        P.kb_spline = F.cs.kb_spline; P.kb_total = kb_total;
        P.n_otiles = F.n_otiles; P.n_ohalves = L.plan.n_otiles * 2;
        P.n_blocks64 = L.plan.kb_total;
        P.kb_o = (s.O + BLOCK_K - 1) / BLOCK_K;
        P.kb_o_chunk = dx_chunk_kb();
        P.n_fgroups = (s.I + 255) / 256;
        P.has_base = has_base ? 1 : 0;
        P.n_items = ((s.N + BLOCK_M - 1) / BLOCK_M) * P.n_fgroups;
        P.vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(gx) & 15) == 0);
        P.ti = ti;
        const int blocks = (int)(P.n_items < sm_count() ? P.n_items : sm_count());
#define KAN_DX(NT, W)                                                                                          \
    do {                                                                                                      \
        e = ensure_dynamic_smem<tc_bwd_input_kernel<NT, W>>((int)DX_SMEM_BYTES);                              \
        if (e == cudaSuccess)                                                                                 \
            tc_bwd_input_kernel<NT, W><<<blocks, TC_THREADS, DX_SMEM_BYTES, st>>>(x, tab, dyimg, wimg, gx,    \
                                                                                   status, P);                \
    } while (0)
        if (ti.cpf == 1) {
            if (split_terms == 3) KAN_DX(3, false); else KAN_DX(1, false);
        } else {
            // without a base branch nothing stores gx first: the spline sub-tiles add to zeros
            if (!has_base && (e = cudaMemsetAsync(gx, 0, (size_t)s.N * s.I * sizeof(float), st)) != cudaSuccess)
                return e;
            if (split_terms == 3) KAN_DX(3, true); else KAN_DX(1, true);
        }
#undef KAN_DX
        if (e != cudaSuccess) return e;
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace kanb200
