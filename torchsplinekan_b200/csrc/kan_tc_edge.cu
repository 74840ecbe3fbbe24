// Edge statistic of the activation regulariser on the tensor cores, straight from x:
//
//     a[o, i] = (1/N) sum_n | s(x[n,i]) bw[o,i] + sum_r B_r(x[n,i]) W[o,i,r] |
//
// For ONE input feature the inner expression is a small matrix product
//     phi_i [outputs, samples] = Wop_i [outputs, 16] . Aop_i [samples, 16]^T
// whose 16 columns are the feature's 8 spline slots, its base value s(x) and 7 zeros: exactly one
// K = 16 step of tcgen05.mma.  The sample-side operand is evaluated from x by producer warps (the
// same window evaluation and hi/lo bf16 split as the layer kernels, three MMAs per product), the
// weight-side operand is a pre-swizzled image fetched by one bulk copy per work item, phi lands in
// tensor memory with OUTPUTS on the lanes and SAMPLES on the columns, and the epilogue warps add up
// |phi| along their own row: no shuffles, no atomics, phi and the basis are never stored.
//
// Work item = (group of 4 features, pair of 128-output tiles, range of samples).  Per 256-sample
// tile the producers write one operand tile (256 rows x 4 features x 16 slots), the MMA thread
// issues 4 features x 2 output tiles x 3 terms MMAs into two alternating 256-column accumulators,
// and the epilogue threads keep one running sum per (output row, feature, output tile).  Partial
// sums go to per-(sample range, column half) slabs that a second kernel adds in a fixed order.
//
// Limits: float32, G + k <= 8 (one 8-slot chunk per feature).  Every wait is bounded.
#include "kan_tc_common.cuh"

namespace kanb200 {

namespace {

constexpr int EDGE_PRODUCER_WARPS = 8, EDGE_EPILOGUE_WARPS = 8;
constexpr int EDGE_PRODUCERS = EDGE_PRODUCER_WARPS * 32;          // one sample row each
constexpr int EDGE_EPILOGUE = EDGE_EPILOGUE_WARPS * 32;           // 128 rows x 2 column halves
constexpr int EDGE_MMA_WARP = EDGE_PRODUCER_WARPS + EDGE_EPILOGUE_WARPS;
constexpr int EDGE_THREADS = (EDGE_MMA_WARP + 2) * 32;
constexpr int EDGE_TN = 256;                                      // samples per tile = accumulator columns
constexpr int EDGE_FQ = 4;                                        // features per operand tile (4 x 16 slots = 128 B)
constexpr int EDGE_OT = 128;                                      // outputs per tile = accumulator rows
constexpr int EDGE_MAX_OTILES = 2;                                // output tiles per work item

constexpr uint32_t EDGE_A_TILE = EDGE_TN * 128;                   // 32 KB: 256 samples x 128 B
constexpr uint32_t EDGE_A_STAGE = 2 * EDGE_A_TILE;                // hi + lo
constexpr int EDGE_A_STAGES = 2;
constexpr uint32_t EDGE_W_TILE = EDGE_OT * 128;                   // 16 KB: 128 outputs x 128 B
constexpr uint32_t EDGE_W_SLOT = 2 * EDGE_W_TILE;                 // hi + lo of one output tile
constexpr uint32_t EDGE_SMEM_A = 0;
constexpr uint32_t EDGE_SMEM_W = EDGE_SMEM_A + EDGE_A_STAGES * EDGE_A_STAGE;
constexpr uint32_t EDGE_SMEM_CTRL = EDGE_SMEM_W + EDGE_MAX_OTILES * EDGE_W_SLOT;
constexpr uint32_t EDGE_SMEM_BYTES = EDGE_SMEM_CTRL + 256 + TAB_SMEM_FLOATS * 4;
static_assert(EDGE_SMEM_BYTES <= 232448, "edge kernel shared memory exceeds 227 KB");

struct EdgeCtrl {
    uint64_t fullA[EDGE_A_STAGES], emptyA[EDGE_A_STAGES];
    uint64_t fullW, emptyW;
    uint64_t accFull[2], accEmpty[2];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(EdgeCtrl) <= 256, "control block too large");

struct EdgePlanTc {
    int n_quads;           // groups of 4 features
    int n_otiles;          // tiles of 128 outputs
    int n_opairs;          // work-item groups of up to 2 output tiles
    int splits;            // sample ranges
    int64_t tiles_total;   // 256-sample tiles
    int64_t tiles_per_split;
    __host__ __device__ int64_t n_items() const { return (int64_t)n_quads * n_opairs * splits; }
    __host__ __device__ int n_slabs() const { return splits * 2; }
};

// Weight-side operand image: for every (output tile of 128, group of 4 features) a hi tile and a lo
// tile of 16 KB each, byte-for-byte the 128-byte-swizzled K-major shared-memory operand: row =
// output, 128 B = 4 features x [8 spline slots | base weight, 7 zeros].
__global__ void pack_edge_weights_kernel(const float* __restrict__ W, const float* __restrict__ bw,
                                         const float* __restrict__ edge_scale, float scale,
                                         uint8_t* __restrict__ img, int O, int I, int R, int n_quads, int n_otiles) {
    const int64_t chunks = (int64_t)n_otiles * n_quads * EDGE_OT * 8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < chunks;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int cc = (int)(idx & 7);
        int64_t rest = idx >> 3;
        const int rr = (int)(rest % EDGE_OT);
        rest /= EDGE_OT;
        const int fq = (int)(rest % n_quads);
        const int ot = (int)(rest / n_quads);
        const int o = ot * EDGE_OT + rr, f = fq * EDGE_FQ + (cc >> 1);
        float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (o < O && f < I) {
            const size_t oi = (size_t)o * I + f;
            if ((cc & 1) == 0) {
                for (int e = 0; e < 8; ++e)
                    if (e < R) w[e] = W[oi * R + e];
            } else if (bw) {
                w[0] = bw[oi];
            }
            if (edge_scale) {
                const float sc = edge_scale[oi] * scale;
#pragma unroll
                for (int e = 0; e < 8; ++e) w[e] *= sc;
            }
        }
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split2(w[2 * e], w[2 * e + 1], h[e], l[e]);
        uint8_t* tile = img + ((size_t)ot * n_quads + fq) * (size_t)EDGE_W_SLOT;
        const uint32_t off = sw128_chunk_offset((uint32_t)rr, (uint32_t)cc);
        *reinterpret_cast<uint4*>(tile + off) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(tile + EDGE_W_TILE + off) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

template <int NTERMS>
__global__ void __launch_bounds__(EDGE_THREADS, 1)
tc_edge_fwd_kernel(const float* __restrict__ x, const float* __restrict__ sbase_val, const float* __restrict__ tab,
                   const uint8_t* __restrict__ wimg, float* __restrict__ partial, int* __restrict__ status,
                   int64_t N, int I, int O, int has_base, EdgePlanTc plan, TabInfo ti, int vec_x) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    EdgeCtrl* ctrl = reinterpret_cast<EdgeCtrl*>(smem + EDGE_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + EDGE_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool shared_grid = grid_is_shared(tab, I, ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < ti.fs) stab[threadIdx.x] = tab[threadIdx.x];

    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) report_status(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < EDGE_A_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullA[s]), EDGE_PRODUCERS);
            mbar_init(smem_u32(&ctrl->emptyA[s]), 1);
        }
        mbar_init(smem_u32(&ctrl->fullW), 1);
        mbar_init(smem_u32(&ctrl->emptyW), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctrl->accFull[s]), 1);
            mbar_init(smem_u32(&ctrl->accEmpty[s]), EDGE_EPILOGUE);
        }
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == EDGE_MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    const int64_t n_items = plan.n_items();

    // item -> (sample range, output pair, feature group); consecutive items share the samples
    auto decode = [&](int64_t item, int& sp, int& op, int& fq) {
        fq = (int)(item % plan.n_quads);
        const int64_t rest = item / plan.n_quads;
        op = (int)(rest % plan.n_opairs);
        sp = (int)(rest / plan.n_opairs);
    };
    auto tile_range = [&](int sp, int64_t& t0, int64_t& t1) {
        t0 = (int64_t)sp * plan.tiles_per_split;
        t1 = t0 + plan.tiles_per_split;
        if (t1 > plan.tiles_total) t1 = plan.tiles_total;
    };
    auto otiles_of = [&](int op) { return (plan.n_otiles - EDGE_MAX_OTILES * op) >= EDGE_MAX_OTILES ? EDGE_MAX_OTILES : 1; };

    if (warp < EDGE_PRODUCER_WARPS) {
        // ===== producers: thread = one sample row of the tile, 4 features each =====
        const int row = threadIdx.x;                      // 0 .. 255
        uint32_t it = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int sp, op, fq;
            decode(item, sp, op, fq);
            int64_t t0, t1;
            tile_range(sp, t0, t1);
            const int f0 = fq * EDGE_FQ;
            for (int64_t t = t0; t < t1; ++t, ++it) {
                const uint32_t stage = it % EDGE_A_STAGES;
                const uint32_t a_hi = sbase + EDGE_SMEM_A + stage * EDGE_A_STAGE;
                const uint32_t a_lo = a_hi + EDGE_A_TILE;
                const int64_t n = t * EDGE_TN + row;
                const bool row_ok = n < N;
                float xv[EDGE_FQ] = {0.f, 0.f, 0.f, 0.f}, sv[EDGE_FQ] = {0.f, 0.f, 0.f, 0.f};
                if (row_ok) {
                    const float* xr = x + (size_t)n * I + f0;
                    if (vec_x && f0 + EDGE_FQ <= I) {
                        const float4 v = __ldg(reinterpret_cast<const float4*>(xr));
                        xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                    } else {
#pragma unroll
                        for (int q = 0; q < EDGE_FQ; ++q)
                            if (f0 + q < I) xv[q] = __ldg(xr + q);
                    }
                    if (has_base) {
                        if (sbase_val) {
                            const float* sr = sbase_val + (size_t)n * I + f0;
#pragma unroll
                            for (int q = 0; q < EDGE_FQ; ++q)
                                if (f0 + q < I) sv[q] = __ldg(sr + q);
                        } else {
#pragma unroll
                            for (int q = 0; q < EDGE_FQ; ++q) sv[q] = silu_fast(xv[q]);
                        }
                    }
                }
                uint4 hi[EDGE_FQ], lo[EDGE_FQ];
                uint32_t bh[EDGE_FQ], bl[EDGE_FQ];
#pragma unroll
                for (int q = 0; q < EDGE_FQ; ++q) {
                    const int f = f0 + q;
                    const float* ft = tab + (size_t)(f < I ? f : I - 1) * ti.fs;
                    const Window w = shared_grid ? eval_window<SPLIT, true, false>(stab, ti, xv[q])
                                                 : eval_window<SPLIT, false, false>(ft, ti, xv[q]);
                    place_window<SPLIT>(w, 0, hi[q], lo[q]);
                    if (!(row_ok && f < I)) {
                        hi[q] = make_uint4(0, 0, 0, 0);
                        lo[q] = hi[q];
                        sv[q] = 0.f;
                    }
                    uint32_t h2, l2;
                    split2(sv[q], 0.0f, h2, l2);
                    bh[q] = h2;
                    bl[q] = SPLIT ? l2 : 0u;
                }
                if (!mbar_wait(smem_u32(&ctrl->emptyA[stage]), ((it / EDGE_A_STAGES) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
#pragma unroll
                for (int q = 0; q < EDGE_FQ; ++q) {
                    const uint32_t off0 = sw128_chunk_offset((uint32_t)row, (uint32_t)(2 * q));
                    const uint32_t off1 = sw128_chunk_offset((uint32_t)row, (uint32_t)(2 * q + 1));
                    st_shared_v4(a_hi + off0, hi[q]);
                    st_shared_v4(a_hi + off1, make_uint4(bh[q], 0, 0, 0));
                    if (SPLIT) {
                        st_shared_v4(a_lo + off0, lo[q]);
                        st_shared_v4(a_lo + off1, make_uint4(bl[q], 0, 0, 0));
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullA[stage]));
            }
        }
    } else if (warp < EDGE_MMA_WARP) {
        // ===== epilogue: thread = one output row of the accumulator, one half of its columns =====
        const int e = warp - EDGE_PRODUCER_WARPS;          // 0 .. 7
        const int quad = warp & 3;                         // TMEM lane quadrant of this warp
        const int half = e >> 2;                           // columns [128 half, 128 half + 128)
        const int orow = quad * 32 + lane;
        uint32_t job = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int sp, op, fq;
            decode(item, sp, op, fq);
            int64_t t0, t1;
            tile_range(sp, t0, t1);
            const int n_ot = otiles_of(op);
            float total[EDGE_MAX_OTILES][EDGE_FQ];
#pragma unroll
            for (int j = 0; j < EDGE_MAX_OTILES; ++j)
#pragma unroll
                for (int q = 0; q < EDGE_FQ; ++q) total[j][q] = 0.f;
            for (int64_t t = t0; t < t1 && ok; ++t) {
#pragma unroll
                for (int j = 0; j < EDGE_MAX_OTILES; ++j) {
                    if (j >= n_ot) break;
#pragma unroll
                    for (int q = 0; q < EDGE_FQ; ++q, ++job) {
                        const uint32_t buf = job & 1u;
                        if (!mbar_wait(smem_u32(&ctrl->accFull[buf]), (job >> 1) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            uint32_t r[32];
                            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * EDGE_TN + half * 128 + c * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int v = 0; v < 32; ++v) part[v & 3] += fabsf(__uint_as_float(r[v]));
                        }
                        total[j][q] += (part[0] + part[1]) + (part[2] + part[3]);
                        tc_fence_before_sync();
                        mbar_arrive(smem_u32(&ctrl->accEmpty[buf]));
                    }
                    if (!ok) break;
                }
            }
            if (!ok) break;
            // slab (sample range, column half) of the per-edge partial sums
            float* slab = partial + ((size_t)sp * 2 + half) * ((size_t)O * I);
#pragma unroll
            for (int j = 0; j < EDGE_MAX_OTILES; ++j) {
                if (j >= n_ot) break;
                const int o = (op * EDGE_MAX_OTILES + j) * EDGE_OT + orow;
                if (o >= O) continue;
#pragma unroll
                for (int q = 0; q < EDGE_FQ; ++q) {
                    const int f = fq * EDGE_FQ + q;
                    if (f < I) slab[(size_t)o * I + f] = total[j][q];
                }
            }
        }
    } else if (warp == EDGE_MMA_WARP) {
        if (lane == 0) {
            // ===== MMA issue: D[o, n] = Wop[o, 16] Aop[n, 16]^T per feature and output tile =====
            constexpr uint32_t idesc = make_idesc_bf16(EDGE_TN, false, false);
            constexpr uint64_t dbase = make_sdesc_sw128(16, 1024);
            uint32_t it = 0, job = 0, n_item = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_item) {
                int sp, op, fq;
                decode(item, sp, op, fq);
                int64_t t0, t1;
                tile_range(sp, t0, t1);
                const int n_ot = otiles_of(op);
                if (!mbar_wait(smem_u32(&ctrl->fullW), n_item & 1u, abort_flag)) break;
                tc_fence_after_sync();
                for (int64_t t = t0; t < t1 && ok; ++t, ++it) {
                    const uint32_t stage = it % EDGE_A_STAGES;
                    const uint32_t a_hi = sbase + EDGE_SMEM_A + stage * EDGE_A_STAGE;
                    const uint32_t a_lo = a_hi + EDGE_A_TILE;
                    if (!mbar_wait(smem_u32(&ctrl->fullA[stage]), (it / EDGE_A_STAGES) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    for (int j = 0; j < n_ot && ok; ++j) {
                        const uint32_t w_hi = sbase + EDGE_SMEM_W + j * EDGE_W_SLOT;
                        const uint32_t w_lo = w_hi + EDGE_W_TILE;
                        for (int q = 0; q < EDGE_FQ; ++q, ++job) {
                            const uint32_t buf = job & 1u;
                            if (!mbar_wait(smem_u32(&ctrl->accEmpty[buf]), ((job >> 1) & 1u) ^ 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t d_tmem = tmem_base + buf * EDGE_TN;
                            mma_f16_ss(d_tmem, sdesc_at(dbase, w_hi + q * 32), sdesc_at(dbase, a_hi + q * 32), idesc, 0u);
                            if (SPLIT) {
                                mma_f16_ss(d_tmem, sdesc_at(dbase, w_lo + q * 32), sdesc_at(dbase, a_hi + q * 32), idesc, 1u);
                                mma_f16_ss(d_tmem, sdesc_at(dbase, w_hi + q * 32), sdesc_at(dbase, a_lo + q * 32), idesc, 1u);
                            }
                            mma_commit(smem_u32(&ctrl->accFull[buf]));
                        }
                    }
                    if (!ok) break;
                    mma_commit(smem_u32(&ctrl->emptyA[stage]));
                }
                if (!ok) break;
                mma_commit(smem_u32(&ctrl->emptyW));
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk copies: the weight tiles of an item, once per item =====
            uint32_t n_item = 0;
            for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x, ++n_item) {
                int sp, op, fq;
                decode(item, sp, op, fq);
                const int n_ot = otiles_of(op);
                if (!mbar_wait(smem_u32(&ctrl->emptyW), (n_item & 1u) ^ 1u, abort_flag)) break;
                const uint32_t bar = smem_u32(&ctrl->fullW);
                mbar_arrive_expect_tx(bar, (uint32_t)n_ot * EDGE_W_SLOT);
                for (int j = 0; j < n_ot; ++j) {
                    const int ot = op * EDGE_MAX_OTILES + j;
                    const uint8_t* src = wimg + ((size_t)ot * plan.n_quads + fq) * (size_t)EDGE_W_SLOT;
                    bulk_g2s(sbase + EDGE_SMEM_W + j * EDGE_W_SLOT, src, EDGE_W_SLOT, bar);
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
    if (warp == EDGE_MMA_WARP) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

__global__ void edge_sum_slabs_kernel(const float* __restrict__ partial, float* __restrict__ a, int64_t elems,
                                      int slabs, float scale) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < elems;
         e += (int64_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < slabs; ++s) v += partial[(size_t)s * elems + e];
        a[e] = v * scale;
    }
}

EdgePlanTc plan_edge_tc(int64_t N, int I, int O) {
    EdgePlanTc p;
    p.n_quads = (I + EDGE_FQ - 1) / EDGE_FQ;
    p.n_otiles = (O + EDGE_OT - 1) / EDGE_OT;
    p.n_opairs = (p.n_otiles + EDGE_MAX_OTILES - 1) / EDGE_MAX_OTILES;
    p.tiles_total = (N + EDGE_TN - 1) / EDGE_TN;
    const int64_t base_items = (int64_t)p.n_quads * p.n_opairs;
    // enough items for about four rounds of the persistent CTAs, at least two sample tiles each
    int64_t splits = (4 * (int64_t)sm_count() + base_items - 1) / base_items;
    const int64_t max_splits = (p.tiles_total + 1) / 2;
    if (splits > max_splits) splits = max_splits;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    p.tiles_per_split = (p.tiles_total + splits - 1) / splits;
    p.splits = (int)((p.tiles_total + p.tiles_per_split - 1) / p.tiles_per_split);
    return p;
}


// ===========================================================================================
// Backward of the edge statistic on the tensor cores.
//
// With phi_i[o, n] as above and S_i = sign(phi_i) (exact in bf16: -1, +1),
//     dW[o,i,r']  = (ga[o,i] / N) sum_n S_i[o,n] A_i[n,r']          r' = 8 spline slots | base value
//     gx[n,i]     = sum_r' dA_i[n,r'] sum_o S_i[o,n] (ga[o,i] / N) W[o,i,r']
// are two more small products per feature, chained behind the first through shared memory:
//     GEMM1  phi [o 128, n 128] = Wop [o,16] Aop[n,16]^T            three terms (hi/lo split of both)
//     sign   16 warps read phi from tensor memory and write S as a bf16 tile [o][n]
//     GEMM2  G   [o 128, 32]    += S[o, n] [A_hi | A_lo][n, 32]     S K-major; the SAME sample tile read
//                                                                   MN-major, 32 columns per feature
//     GEMM3  D3  [n 128, 32]    += S^T[n, o] [Wg_hi | Wg_lo][o, 32] the S tile read MN-major, Wg = ga W / N
// An MMA instruction costs its issuing thread about 64 cycles however few columns it has (measured,
// kanb200_selftest_umma_rate), so the hi and lo parts of an operand sit side by side in the
// 128-byte rows (a row = 2 features x [16 hi | 16 lo]) and one N = 32 instruction serves both; the
// epilogues add the two halves.  GEMM1 / GEMM2 and GEMM3 are issued by two different threads.
// G stays in tensor memory over all sample tiles of a work item (at most 8 tiles = 1024 samples per
// accumulation chain), D3 over the output tiles of one sample tile.  At the end of an item the sign
// warps scale G into per-split slabs; per sample tile four more warps contract D3 with the basis
// derivatives of x (from the polynomial table) into gx.  Nothing of size [N, O, I] or [N, I, R] is
// ever stored.  A work item = (range of samples, group of 4 features, tile of 128 outputs); with two
// output tiles (129 .. 256 outputs) the two items of a sample tile each add their share to a
// zero-filled gx (red.add of exactly two terms: the result does not depend on the order).
// Tensor memory: phi 2 x 128 columns, G 4 x 32, D3 4 x 32.
// ===========================================================================================
constexpr int EB_TN = 128;                                        // samples per tile
constexpr int EB_PRODUCER_WARPS = 4, EB_SIGN_WARPS = 16, EB_GX_WARPS = 4;
constexpr int EB_PRODUCERS = EB_PRODUCER_WARPS * 32, EB_SIGNERS = EB_SIGN_WARPS * 32, EB_GXERS = EB_GX_WARPS * 32;
constexpr int EB_MMA_WARP = EB_PRODUCER_WARPS + EB_SIGN_WARPS + EB_GX_WARPS;      // GEMM1, GEMM2
constexpr int EB_MMA3_WARP = EB_MMA_WARP + 1;                                     // GEMM3
constexpr int EB_THREADS = (EB_MMA_WARP + 3) * 32;
constexpr int EB_MAX_CHAIN_TILES = 8;
constexpr uint32_t EB_A_TILE = EB_TN * 128;                       // 16 KB: 128 samples x 2 features x [hi | lo]
constexpr uint32_t EB_A_STAGE = 2 * EB_A_TILE;                    // features 0-1, features 2-3
constexpr uint32_t EB_S_BLOCK = EDGE_OT * 128;                    // 16 KB: 128 outputs x 64 samples
constexpr uint32_t EB_S_TILE = 2 * EB_S_BLOCK;                    // 32 KB: 128 outputs x 128 samples
constexpr uint32_t EB_SMEM_A = 0;                                 // two stages of the sample-side operand
constexpr uint32_t EB_SMEM_S = EB_SMEM_A + 2 * EB_A_STAGE;        // two sign tiles: conversion runs one unit ahead
constexpr uint32_t EB_SMEM_W = EB_SMEM_S + 2 * EB_S_TILE;
constexpr uint32_t EB_SMEM_WG = EB_SMEM_W + EDGE_W_SLOT;
constexpr uint32_t EB_SMEM_XS = EB_SMEM_WG + EDGE_W_SLOT;          // float32 x of the two operand stages: [2][128][4]
constexpr uint32_t EB_SMEM_WROWS = EB_SMEM_XS + 2 * EB_TN * EDGE_FQ * 4;   // float32 weights of the item: [128][4][12]
constexpr uint32_t EB_WROW_FLOATS = 12;                           // 8 coefficients, base weight, re-check bound, 2 unused
constexpr uint32_t EB_SMEM_CTRL = EB_SMEM_WROWS + EDGE_OT * EDGE_FQ * EB_WROW_FLOATS * 4;
constexpr uint32_t EB_SMEM_BYTES = EB_SMEM_CTRL + 256 + TAB_SMEM_FLOATS * 4;
static_assert(EB_SMEM_BYTES <= 232448, "edge backward kernel shared memory exceeds 227 KB");
constexpr uint32_t EB_TMEM_G = 256, EB_TMEM_D3 = 384;

struct EdgeBwdCtrl {
    uint64_t fullA[2], emptyA[2];
    uint64_t fullW, emptyW;
    uint64_t phiFull[2], phiEmpty[2];     // accumulator b, sign tile b and sign group b belong together
    uint64_t sFull[2], sEmpty[2];
    uint64_t gFull, gEmpty;
    uint64_t d3Full, d3Empty;
    uint64_t wrFull, wrFree;              // float32 weight rows of the item (sign warps among themselves)
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(EdgeBwdCtrl) <= 256, "control block too large");

struct EdgeBwdPlan {
    int n_quads, n_otiles, splits;
    int64_t tiles_total, tiles_per_split;
    __host__ __device__ int64_t n_items() const { return (int64_t)n_quads * n_otiles * splits; }
};

// Weight-side operand image of the backward kernel: per (output tile of 128, group of 4 features) two
// tiles of 16 KB (features 0-1, features 2-3), rows of 128 B = 2 features x [hi: 8 spline slots,
// base weight, 7 zeros | lo: the same], 128-byte-swizzled.  edge_scale (ga) and scale (1 / N), when
// given, are folded in (the operand of GEMM3).
__global__ void pack_edge_weights_pairs_kernel(const float* __restrict__ W, const float* __restrict__ bw,
                                               const float* __restrict__ edge_scale, float scale,
                                               uint8_t* __restrict__ img, int O, int I, int R, int n_quads,
                                               int n_otiles) {
    const int64_t units = (int64_t)n_otiles * n_quads * EDGE_OT * EDGE_FQ;      // (tile, group, row, feature)
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < units;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int q = (int)(idx & 3);
        int64_t rest = idx >> 2;
        const int rr = (int)(rest % EDGE_OT);
        rest /= EDGE_OT;
        const int fq = (int)(rest % n_quads);
        const int ot = (int)(rest / n_quads);
        const int o = ot * EDGE_OT + rr, f = fq * EDGE_FQ + q;
        float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float b = 0.f;
        if (o < O && f < I) {
            const size_t oi = (size_t)o * I + f;
            const float sc = edge_scale ? edge_scale[oi] * scale : 1.0f;
            for (int e = 0; e < 8; ++e)
                if (e < R) w[e] = W[oi * R + e] * sc;
            if (bw) b = bw[oi] * sc;
        }
        uint32_t h[4], l[4], bh, bl;
#pragma unroll
        for (int e = 0; e < 4; ++e) split2(w[2 * e], w[2 * e + 1], h[e], l[e]);
        split2(b, 0.0f, bh, bl);
        uint8_t* tile = img + ((size_t)ot * n_quads + fq) * (size_t)EDGE_W_SLOT + (size_t)(q >> 1) * EDGE_W_TILE;
        const uint32_t c0 = (uint32_t)(4 * (q & 1));
        *reinterpret_cast<uint4*>(tile + sw128_chunk_offset((uint32_t)rr, c0)) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(tile + sw128_chunk_offset((uint32_t)rr, c0 + 1)) = make_uint4(bh, 0, 0, 0);
        *reinterpret_cast<uint4*>(tile + sw128_chunk_offset((uint32_t)rr, c0 + 2)) = make_uint4(l[0], l[1], l[2], l[3]);
        *reinterpret_cast<uint4*>(tile + sw128_chunk_offset((uint32_t)rr, c0 + 3)) = make_uint4(bl, 0, 0, 0);
    }
}

__global__ void __launch_bounds__(EB_THREADS, 1)
tc_edge_bwd_kernel(const float* __restrict__ x, const float* __restrict__ tab, const uint8_t* __restrict__ wimg,
                   const uint8_t* __restrict__ wgimg, const float* __restrict__ ga, const float* __restrict__ Wf,
                   const float* __restrict__ bwf, float* __restrict__ slabs, float* __restrict__ gx,
                   int* __restrict__ status, int64_t N, int I, int O, int R, EdgeBwdPlan plan, TabInfo ti,
                   int vec_x, int recheck) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    EdgeBwdCtrl* ctrl = reinterpret_cast<EdgeBwdCtrl*>(smem + EB_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + EB_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool need_gx = gx != nullptr;
    const int has_base = bwf != nullptr;
    float* xs = reinterpret_cast<float*>(smem + EB_SMEM_XS);
    float* wrows = reinterpret_cast<float*>(smem + EB_SMEM_WROWS);
    const bool shared_grid = grid_is_shared(tab, I, ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < ti.fs) stab[threadIdx.x] = tab[threadIdx.x];

    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) report_status(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        const uint32_t issuers = need_gx ? 2u : 1u;                      // threads whose MMAs read S and W
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctrl->sFull[s]), EB_SIGNERS / 2);      // one group of sign warps each
            mbar_init(smem_u32(&ctrl->sEmpty[s]), issuers);
            mbar_init(smem_u32(&ctrl->phiFull[s]), 1);
            mbar_init(smem_u32(&ctrl->phiEmpty[s]), EB_SIGNERS / 2);
            mbar_init(smem_u32(&ctrl->fullA[s]), EB_PRODUCERS);
            mbar_init(smem_u32(&ctrl->emptyA[s]), 1);
        }
        mbar_init(smem_u32(&ctrl->d3Full), 1);
        mbar_init(smem_u32(&ctrl->d3Empty), EB_GXERS);
        mbar_init(smem_u32(&ctrl->wrFull), EB_SIGNERS);
        mbar_init(smem_u32(&ctrl->wrFree), EB_SIGNERS);
        mbar_init(smem_u32(&ctrl->fullW), 1);
        mbar_init(smem_u32(&ctrl->emptyW), issuers);
        mbar_init(smem_u32(&ctrl->gFull), 1);
        mbar_init(smem_u32(&ctrl->gEmpty), EB_SIGNERS);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == EB_MMA_WARP) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    const int64_t n_items = plan.n_items();
    const bool add_gx = plan.n_otiles > 1;              // two items contribute to every gx entry

    // item -> (sample range, output tile, feature group); consecutive items share the samples
    auto decode3 = [&](int64_t item, int& sp, int& ot, int& fq) {
        fq = (int)(item % plan.n_quads);
        const int64_t rest = item / plan.n_quads;
        ot = (int)(rest % plan.n_otiles);
        sp = (int)(rest / plan.n_otiles);
    };
    auto decode = [&](int64_t item, int& sp, int& fq) {
        int ot;
        decode3(item, sp, ot, fq);
    };
    auto tile_range = [&](int sp, int64_t& t0, int64_t& t1) {
        t0 = (int64_t)sp * plan.tiles_per_split;
        t1 = t0 + plan.tiles_per_split;
        if (t1 > plan.tiles_total) t1 = plan.tiles_total;
    };
    // shared-memory address of feature q's [hi | lo] columns inside a tile pair that starts at `base`
    auto pair_addr = [](uint32_t base, uint32_t tile_bytes, int q) -> uint32_t {
        return base + (uint32_t)(q >> 1) * tile_bytes + (uint32_t)(q & 1) * 64u;
    };

    if (warp < EB_PRODUCER_WARPS) {
        // ===== producers: thread = one sample row, its four features in two passes =====
        const int row = threadIdx.x;                                            // 0 .. 127
        uint32_t it = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int sp, fq;
            decode(item, sp, fq);
            int64_t t0, t1;
            tile_range(sp, t0, t1);
            for (int64_t t = t0; t < t1; ++t, ++it) {
                const int64_t n = t * EB_TN + row;
                const bool row_ok = n < N;
                bool waited = false;
#pragma unroll 1
                for (int pr = 0; pr < 2; ++pr) {
                    const uint32_t a_tile = sbase + EB_SMEM_A + (it & 1u) * EB_A_STAGE + (uint32_t)pr * EB_A_TILE;
                    const int f0 = fq * EDGE_FQ + 2 * pr;
                    float xv[2] = {0.f, 0.f};
                    if (row_ok) {
                        const float* xr = x + (size_t)n * I + f0;
                        if (vec_x && f0 + 2 <= I) {
                            const float2 v = __ldg(reinterpret_cast<const float2*>(xr));
                            xv[0] = v.x; xv[1] = v.y;
                        } else {
#pragma unroll
                            for (int q = 0; q < 2; ++q)
                                if (f0 + q < I) xv[q] = __ldg(xr + q);
                        }
                    }
                    uint4 hi[2], lo[2];
                    uint32_t bh[2], bl[2];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int f = f0 + q;
                        const float* ft = tab + (size_t)(f < I ? f : I - 1) * ti.fs;
                        const Window w = shared_grid ? eval_window<true, true, false>(stab, ti, xv[q])
                                                     : eval_window<true, false, false>(ft, ti, xv[q]);
                        place_window<true>(w, 0, hi[q], lo[q]);
                        float sv = has_base ? silu_fast(xv[q]) : 0.f;
                        if (!(row_ok && f < I)) {
                            hi[q] = make_uint4(0, 0, 0, 0);
                            lo[q] = hi[q];
                            sv = 0.f;
                        }
                        split2(sv, 0.0f, bh[q], bl[q]);
                    }
                    if (!waited && !mbar_wait(smem_u32(&ctrl->emptyA[it & 1u]), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    waited = true;
                    *reinterpret_cast<float2*>(xs + ((it & 1u) * EB_TN + row) * EDGE_FQ + 2 * pr) = make_float2(xv[0], xv[1]);
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const uint32_t c0 = (uint32_t)(4 * q);
                        st_shared_v4(a_tile + sw128_chunk_offset((uint32_t)row, c0), hi[q]);
                        st_shared_v4(a_tile + sw128_chunk_offset((uint32_t)row, c0 + 1), make_uint4(bh[q], 0, 0, 0));
                        st_shared_v4(a_tile + sw128_chunk_offset((uint32_t)row, c0 + 2), lo[q]);
                        st_shared_v4(a_tile + sw128_chunk_offset((uint32_t)row, c0 + 3), make_uint4(bl[q], 0, 0, 0));
                    }
                }
                if (!ok) break;
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullA[it & 1u]));
            }
        }
    } else if (warp < EB_PRODUCER_WARPS + EB_SIGN_WARPS) {
        // ===== sign warps: two groups of eight; group g converts the units with job parity g into sign
        // tile g, so one conversion overlaps the products that read the other tile; thread = one output
        // row, 64 samples.  sign(phi) as bf16 is the float's sign bit over the pattern of 1.0 (0x3F80);
        // an exact zero counts as +1, which only matters for edges whose weights are all zero (the
        // finalize kernel writes their gradients as zero, and their scaled weights add nothing to gx).
        // The split-bf16 product gives phi to about 2^-17 of its terms (measured: 4e-6 .. 7e-6 of the
        // largest); with `recheck`, where |phi| is below 2e-5 of a bound on them, max_r |W_r| + 2 |bw|, the
        // thread evaluates that one phi again in float32 -- x of the tile and the item's weight rows are
        // kept in shared memory for that -- so the signs are those of a float32 evaluation (some tens of
        // values per million take this path) =====
        const int e = warp - EB_PRODUCER_WARPS;            // 0 .. 15
        const int quad = warp & 3;
        const int half = e >> 3;                           // the group
        const int ch = (e >> 2) & 1;                       // samples [64 ch, 64 ch + 64)
        const int orow = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t row_off = (uint32_t)(orow >> 3) * 1024u + (uint32_t)(orow & 7) * 128u, x7 = (uint32_t)(orow & 7);
        const float inv_n = 1.0f / (float)N;
        uint32_t job = 0, n_item = 0, tile_it = 0;
        bool ok = true;
        auto sgn2 = [](uint32_t a, uint32_t b) -> uint32_t {
            return (__byte_perm(a, b, 0x7632) & 0x80008000u) | 0x3F803F80u;
        };
        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_item) {
            int sp, ot, fq;
            decode3(item, sp, ot, fq);
            int64_t t0, t1;
            tile_range(sp, t0, t1);
            const int64_t units = (t1 - t0) * EDGE_FQ;                 // a multiple of 4: job stays even at item starts
            const int o_glob = ot * EDGE_OT + orow;
            float tau2[2] = {0.f, 0.f};                                // this group sees features half, half + 2
            if (recheck) {
                // the item's float32 weight rows: thread (row, column half ch, group) loads feature 2 ch + group
                if (!mbar_wait(smem_u32(&ctrl->wrFree), (n_item & 1u) ^ 1u, abort_flag)) break;   // last item's readers
                {
                    const int q = 2 * ch + half, f = fq * EDGE_FQ + q;
                    float* dst = wrows + ((size_t)orow * EDGE_FQ + q) * EB_WROW_FLOATS;
                    float m = 0.f, b = 0.f;
                    const bool live = o_glob < O && f < I;
                    for (int r = 0; r < 8; ++r) {
                        const float w = (live && r < R) ? __ldg(Wf + ((size_t)o_glob * I + f) * R + r) : 0.f;
                        dst[r] = w;
                        m = fmaxf(m, fabsf(w));
                    }
                    if (live && has_base) b = __ldg(bwf + (size_t)o_glob * I + f);
                    dst[8] = b;
                    dst[9] = (m + 2.0f * fabsf(b)) * 2.0e-5f;
                }
                mbar_arrive(smem_u32(&ctrl->wrFull));
                if (!mbar_wait(smem_u32(&ctrl->wrFull), n_item & 1u, abort_flag)) break;
                tau2[0] = wrows[((size_t)orow * EDGE_FQ + half) * EB_WROW_FLOATS + 9];
                tau2[1] = wrows[((size_t)orow * EDGE_FQ + half + 2) * EB_WROW_FLOATS + 9];
            }
            const uint32_t it0 = tile_it;
            for (int64_t u = half; u < units && ok; u += 2) {
                const uint32_t jb = job + (uint32_t)u;
                const uint32_t sb = (uint32_t)half;                     // == jb & 1
                const int qu = (int)(u & 3);
                const float tau = (qu >> 1) ? tau2[1] : tau2[0];
                if (!mbar_wait(smem_u32(&ctrl->phiFull[sb]), (jb >> 1) & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                if (!mbar_wait(smem_u32(&ctrl->sEmpty[sb]), ((jb >> 1) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t s_blk = sbase + EB_SMEM_S + sb * EB_S_TILE + (uint32_t)ch * EB_S_BLOCK + row_off;
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    uint32_t r[32];
                    tmem_ld_32x32(lane_addr + sb * EB_TN + ch * 64 + h2 * 32, r);
                    tmem_ld_wait();
                    if (h2 == 1) {
                        tc_fence_before_sync();
                        mbar_arrive(smem_u32(&ctrl->phiEmpty[sb]));
                    }
                    if (recheck) {
                        float l4[4] = {3.0e38f, 3.0e38f, 3.0e38f, 3.0e38f};  // smallest |phi| of the 32 values
#pragma unroll
                        for (int c = 0; c < 32; ++c) l4[c & 3] = fminf(l4[c & 3], fabsf(__uint_as_float(r[c])));
                        if (fminf(fminf(l4[0], l4[1]), fminf(l4[2], l4[3])) < tau) {   // rare
                            const float* wrow = wrows + ((size_t)orow * EDGE_FQ + qu) * EB_WROW_FLOATS;
                            const uint32_t stage = (it0 + (uint32_t)(u >> 2)) & 1u;
                            const float* ftab = tab + (size_t)min(fq * EDGE_FQ + qu, I - 1) * ti.fs;
                            uint32_t small = 0u;
#pragma unroll
                            for (int c = 0; c < 32; ++c) small |= (fabsf(__uint_as_float(r[c])) < tau) ? (1u << c) : 0u;
                            while (small) {
                                const int c = __ffs(small) - 1;
                                small &= small - 1u;
                                const float xv = xs[(stage * EB_TN + ch * 64 + h2 * 32 + c) * EDGE_FQ + qu];
                                float v[4];
                                const int s0 = shared_grid ? eval_feature_values<true, false>(stab, ti, xv, v)
                                                           : eval_feature_values<false, false>(ftab, ti, xv, v);
                                float phi = has_base ? silu_fast(xv) * wrow[8] : 0.f;
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj)
                                    if (s0 + jj >= 0 && s0 + jj < 8) phi = fmaf(v[jj], wrow[s0 + jj], phi);
                                const uint32_t bits = __float_as_uint(phi);
#pragma unroll
                                for (int cc = 0; cc < 32; ++cc)
                                    if (cc == c) r[cc] = bits;
                            }
                        }
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        st_shared_v4(s_blk + (((uint32_t)(4 * h2 + c) ^ x7) << 4),
                                     make_uint4(sgn2(r[8 * c], r[8 * c + 1]), sgn2(r[8 * c + 2], r[8 * c + 3]),
                                                sgn2(r[8 * c + 4], r[8 * c + 5]), sgn2(r[8 * c + 6], r[8 * c + 7])));
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->sFull[sb]));
            }
            job += (uint32_t)units;
            tile_it += (uint32_t)(t1 - t0);
            if (!ok) break;
            if (recheck) mbar_arrive(smem_u32(&ctrl->wrFree));
            // the item's parameter-gradient sums: this thread writes feature 2 ch + half of its output row
            if (!mbar_wait(smem_u32(&ctrl->gFull), n_item & 1u, abort_flag)) break;
            tc_fence_after_sync();
            {
                float* slab = slabs + (size_t)sp * ((size_t)O * I * 9);
                const int o = ot * EDGE_OT + orow;
                const int q = 2 * ch + half, f = fq * EDGE_FQ + q;
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + EB_TMEM_G + (uint32_t)q * 32, r);
                tmem_ld_wait();
                if (o < O && f < I) {
                    const float sc = __ldg(ga + (size_t)o * I + f) * inv_n;
                    float* out = slab + ((size_t)o * I + f) * 9;
#pragma unroll
                    for (int c = 0; c < 9; ++c) out[c] = sc * (__uint_as_float(r[c]) + __uint_as_float(r[16 + c]));
                }
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->gEmpty));
        }
    } else if (warp < EB_MMA_WARP) {
        // ===== input-gradient warps: thread = one sample row of the tile =====
        if (need_gx) {
            const int quad = warp & 3;
            const int row = quad * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
            uint32_t it = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int sp, fq;
                decode(item, sp, fq);
                int64_t t0, t1;
                tile_range(sp, t0, t1);
                const int f0 = fq * EDGE_FQ;
                for (int64_t t = t0; t < t1; ++t, ++it) {
                    const int64_t n = t * EB_TN + row;
                    const bool row_ok = n < N;
                    float xv[EDGE_FQ] = {0.f, 0.f, 0.f, 0.f};
                    if (row_ok) {
                        const float* xr = x + (size_t)n * I + f0;
                        if (vec_x && f0 + EDGE_FQ <= I && (I & 3) == 0) {
                            const float4 v = __ldg(reinterpret_cast<const float4*>(xr));
                            xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                        } else {
#pragma unroll
                            for (int q = 0; q < EDGE_FQ; ++q)
                                if (f0 + q < I) xv[q] = __ldg(xr + q);
                        }
                    }
                    if (!mbar_wait(smem_u32(&ctrl->d3Full), it & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    float g[EDGE_FQ];
#pragma unroll
                    for (int q = 0; q < EDGE_FQ; ++q) {
                        const int f = f0 + q;
                        const float* ft = tab + (size_t)(f < I ? f : I - 1) * ti.fs;
                        float d[4];
                        const int s0 = shared_grid ? eval_feature_deriv<true, false>(stab, ti, xv[q], d)
                                                   : eval_feature_deriv<false, false>(ft, ti, xv[q], d);
                        uint32_t r[32];
                        tmem_ld_32x32(lane_addr + EB_TMEM_D3 + (uint32_t)q * 32, r);
                        tmem_ld_wait();
                        float acc = has_base ? (__uint_as_float(r[8]) + __uint_as_float(r[24])) * silu_grad_fast(xv[q]) : 0.f;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const int jj = c - s0;
                            const float dc = jj == 0 ? d[0] : (jj == 1 ? d[1] : (jj == 2 ? d[2] : (jj == 3 ? d[3] : 0.f)));
                            acc = fmaf(__uint_as_float(r[c]) + __uint_as_float(r[16 + c]), dc, acc);
                        }
                        g[q] = acc;
                    }
                    tc_fence_before_sync();
                    mbar_arrive(smem_u32(&ctrl->d3Empty));
                    if (row_ok && add_gx) {
                        float* out = gx + (size_t)n * I + f0;
#pragma unroll
                        for (int q = 0; q < EDGE_FQ; ++q)
                            if (f0 + q < I) atomicAdd(out + q, g[q]);
                    } else if (row_ok) {
                        float* out = gx + (size_t)n * I + f0;
                        if (vec_x && f0 + EDGE_FQ <= I && (I & 3) == 0) {
                            *reinterpret_cast<float4*>(out) = make_float4(g[0], g[1], g[2], g[3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < EDGE_FQ; ++q)
                                if (f0 + q < I) out[q] = g[q];
                        }
                    }
                }
            }
        }
    } else if (warp == EB_MMA_WARP) {
        if (lane == 0) {
            // ===== issuer of GEMM1 and GEMM2 =====
            constexpr uint32_t idesc1 = make_idesc_bf16(EB_TN, false, false);
            constexpr uint32_t idesc2 = make_idesc_bf16(32, false, true);
            constexpr uint64_t d_k = make_sdesc_sw128(16, 1024);          // K-major rows of 128 B
            constexpr uint64_t d_mn = make_sdesc_sw128(8192, 1024);       // MN-major, one group of columns
            uint32_t it = 0, job = 0, n_item = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_item) {
                int sp, fq;
                decode(item, sp, fq);
                int64_t t0, t1;
                tile_range(sp, t0, t1);
                if (!mbar_wait(smem_u32(&ctrl->fullW), n_item & 1u, abort_flag)) break;
                if (!mbar_wait(smem_u32(&ctrl->gEmpty), (n_item & 1u) ^ 1u, abort_flag)) break;
                tc_fence_after_sync();
                auto stage_ready = [&](uint32_t tile_it) -> bool {
                    if (!mbar_wait(smem_u32(&ctrl->fullA[tile_it & 1u]), (tile_it >> 1) & 1u, abort_flag)) return false;
                    tc_fence_after_sync();
                    return true;
                };
                auto gemm1 = [&](uint32_t tile_it, int q, uint32_t jb) -> bool {
                    const uint32_t buf = jb & 1u;
                    if (!mbar_wait(smem_u32(&ctrl->phiEmpty[buf]), ((jb >> 1) & 1u) ^ 1u, abort_flag)) return false;
                    tc_fence_after_sync();
                    const uint32_t w = pair_addr(sbase + EB_SMEM_W, EDGE_W_TILE, q);
                    const uint32_t a = pair_addr(sbase + EB_SMEM_A + (tile_it & 1u) * EB_A_STAGE, EB_A_TILE, q);
                    const uint64_t dw_hi = sdesc_at(d_k, w), da_hi = sdesc_at(d_k, a);
                    const uint32_t d = tmem_base + buf * EB_TN;
                    mma_f16_ss(d, dw_hi, da_hi, idesc1, 0u);
                    mma_f16_ss(d, dw_hi + 2u, da_hi, idesc1, 1u);                  // lo part: 32 bytes on
                    mma_f16_ss(d, dw_hi, da_hi + 2u, idesc1, 1u);
                    mma_commit(smem_u32(&ctrl->phiFull[buf]));
                    return true;
                };
                // units of the item in order (tile, feature); GEMM1 runs one unit ahead of the products
                // that consume the sign tile
                int64_t t = t0;
                int q = 0;
                uint32_t cur_it = it;
                if (!stage_ready(cur_it) || !gemm1(cur_it, 0, job)) break;
                while (true) {
                    int64_t nt = t;
                    int nq = q + 1;
                    if (nq == EDGE_FQ) { nq = 0; ++nt; }
                    const bool has_next = nt < t1, same_tile = nt == t;
                    const uint32_t next_it = cur_it + (same_tile ? 0u : 1u);
                    if (has_next) {
                        if (!same_tile && !stage_ready(next_it)) { ok = false; break; }
                        if (!gemm1(next_it, nq, job + 1)) { ok = false; break; }
                    }
                    const uint32_t sb = job & 1u;
                    if (!mbar_wait(smem_u32(&ctrl->sFull[sb]), (job >> 1) & 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    {   // GEMM2: G[q] (+)= S[o, n] [A_hi | A_lo][n, 32]; addresses advance in 16-byte units
                        const uint32_t s_t = sbase + EB_SMEM_S + sb * EB_S_TILE;
                        const uint32_t d = tmem_base + EB_TMEM_G + (uint32_t)q * 32;
                        const uint64_t ds0 = sdesc_at(d_k, s_t), ds1 = sdesc_at(d_k, s_t + EB_S_BLOCK);
                        const uint64_t db =
                            sdesc_at(d_mn, pair_addr(sbase + EB_SMEM_A + (cur_it & 1u) * EB_A_STAGE, EB_A_TILE, q));
                        const uint32_t first = t > t0 ? 1u : 0u;
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            mma_f16_ss(d, (ks < 4 ? ds0 : ds1) + (uint64_t)((ks & 3) * 2), db + (uint64_t)(ks * 128), idesc2,
                                       ks == 0 ? first : 1u);
                    }
                    mma_commit(smem_u32(&ctrl->sEmpty[sb]));
                    ++job;
                    if (!has_next || !same_tile) mma_commit(smem_u32(&ctrl->emptyA[cur_it & 1u]));
                    if (!has_next) break;
                    t = nt; q = nq; cur_it = next_it;
                }
                if (!ok) break;
                it = cur_it + 1;
                mma_commit(smem_u32(&ctrl->gFull));
                mma_commit(smem_u32(&ctrl->emptyW));
            }
        }
    } else if (warp == EB_MMA3_WARP) {
        if (lane == 0 && need_gx) {
            // ===== issuer of GEMM3: D3[q] (+)= S^T[n, o] [Wg_hi | Wg_lo][o, 32] =====
            constexpr uint32_t idesc3 = make_idesc_bf16(32, true, true);
            constexpr uint64_t d_mn = make_sdesc_sw128(8192, 1024);
            constexpr uint64_t d_mnS = make_sdesc_sw128(EB_S_BLOCK, 1024);  // MN-major, two groups of 64 samples
            uint32_t it = 0, job = 0, n_item = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_item) {
                int sp, fq;
                decode(item, sp, fq);
                int64_t t0, t1;
                tile_range(sp, t0, t1);
                if (!mbar_wait(smem_u32(&ctrl->fullW), n_item & 1u, abort_flag)) break;
                tc_fence_after_sync();
                for (int64_t t = t0; t < t1 && ok; ++t, ++it) {
                    if (!mbar_wait(smem_u32(&ctrl->d3Empty), (it & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    for (int q = 0; q < EDGE_FQ; ++q, ++job) {
                        const uint32_t sb = job & 1u;
                        if (!mbar_wait(smem_u32(&ctrl->sFull[sb]), (job >> 1) & 1u, abort_flag)) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t s_t = sbase + EB_SMEM_S + sb * EB_S_TILE;
                        const uint32_t d = tmem_base + EB_TMEM_D3 + (uint32_t)q * 32;
                        const uint64_t dsT = sdesc_at(d_mnS, s_t);
                        const uint64_t db = sdesc_at(d_mn, pair_addr(sbase + EB_SMEM_WG, EDGE_W_TILE, q));
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            mma_f16_ss(d, dsT + (uint64_t)(ks * 128), db + (uint64_t)(ks * 128), idesc3, ks == 0 ? 0u : 1u);
                        mma_commit(smem_u32(&ctrl->sEmpty[sb]));
                    }
                    if (ok) mma_commit(smem_u32(&ctrl->d3Full));
                }
                if (!ok) break;
                mma_commit(smem_u32(&ctrl->emptyW));
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk copies: the weight tiles of an item (and their ga-scaled twins), once per item =====
            uint32_t n_item = 0;
            for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x, ++n_item) {
                int sp, ot, fq;
                decode3(item, sp, ot, fq);
                if (!mbar_wait(smem_u32(&ctrl->emptyW), (n_item & 1u) ^ 1u, abort_flag)) break;
                const uint32_t bar = smem_u32(&ctrl->fullW);
                mbar_arrive_expect_tx(bar, EDGE_W_SLOT * (need_gx ? 2u : 1u));
                const size_t off = ((size_t)ot * plan.n_quads + fq) * (size_t)EDGE_W_SLOT;
                bulk_g2s(sbase + EB_SMEM_W, wimg + off, EDGE_W_SLOT, bar);
                if (need_gx) bulk_g2s(sbase + EB_SMEM_WG, wgimg + off, EDGE_W_SLOT, bar);
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
    if (warp == EB_MMA_WARP) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

// An edge whose coefficients and base weight are all zero has phi == 0 for every sample, hence
// sign(phi) == 0 and zero gradients (the kernel above counts an exact zero as +1).
__global__ void edge_bwd_finalize_kernel(const float* __restrict__ slabs, int splits, const float* __restrict__ W,
                                         const float* __restrict__ bw, float* __restrict__ dW,
                                         float* __restrict__ dbw, int64_t pairs, int R) {
    const int64_t total = pairs * 9;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t oi = e / 9;
        const int c = (int)(e - oi * 9);
        const bool wanted = c < R ? dW != nullptr : (c == 8 && dbw != nullptr);
        if (!wanted) continue;
        bool live = bw != nullptr && bw[oi] != 0.0f;
        for (int r = 0; r < R && !live; ++r) live = W[oi * R + r] != 0.0f;
        float v = 0.f;
        if (live)
            for (int s = 0; s < splits; ++s) v += slabs[(size_t)s * total + e];
        if (c < R) dW[oi * R + c] = v;
        else dbw[oi] = v;
    }
}

bool g_sign_recheck = true;

EdgeBwdPlan plan_edge_bwd(int64_t N, int I, int O) {
    EdgeBwdPlan p;
    p.n_quads = (I + EDGE_FQ - 1) / EDGE_FQ;
    p.n_otiles = (O + EDGE_OT - 1) / EDGE_OT;
    p.tiles_total = (N + EB_TN - 1) / EB_TN;
    // chains of at most EB_MAX_CHAIN_TILES sample tiles per accumulator, and about four rounds of
    // work items for the persistent blocks
    int64_t splits = (p.tiles_total + EB_MAX_CHAIN_TILES - 1) / EB_MAX_CHAIN_TILES;
    const int64_t base_items = (int64_t)p.n_quads * p.n_otiles;
    const int64_t for_balance = (4 * (int64_t)sm_count() + base_items - 1) / base_items;
    if (splits < for_balance) splits = for_balance;
    if (splits > p.tiles_total) splits = p.tiles_total;
    if (splits < 1) splits = 1;
    p.tiles_per_split = (p.tiles_total + splits - 1) / splits;
    p.splits = (int)((p.tiles_total + p.tiles_per_split - 1) / p.tiles_per_split);
    return p;
}

}  // namespace

bool tc_edge_supported(const LayerShape& s) {
    return s.K >= 1 && s.K <= 3 && s.G >= 1 && s.R() <= 8 && s.N >= 1 && s.I >= 1 && s.O >= 1;
}

size_t tc_edge_workspace(const LayerShape& s) {
    const EdgePlanTc p = plan_edge_tc(s.N, s.I, s.O);
    return kWsHeader + tc_table_bytes(s) + align256((size_t)p.n_otiles * p.n_quads * EDGE_W_SLOT) +
           align256((size_t)p.n_slabs() * s.O * s.I * sizeof(float));
}

// W is the effective coefficient tensor [O, I, R] (scaler already applied); s_val, when given,
// replaces silu(x) as the base value (layers with another base activation); bw == NULL: no base term.
cudaError_t tc_edge_forward(int split_terms, const float* x, const float* s_val, const float* grid, const float* bw,
                            const float* W, float* a, const LayerShape& s, void* ws, size_t ws_bytes,
                            cudaStream_t st) {
    if (!ws || ws_bytes < tc_edge_workspace(s)) return cudaErrorMemoryAllocation;
    const EdgePlanTc p = plan_edge_tc(s.N, s.I, s.O);
    const TabInfo ti = make_tab_info(s.G, s.K);
    int* status = reinterpret_cast<int*>(ws);
    uint8_t* cur = reinterpret_cast<uint8_t*>(ws) + kWsHeader;
    float* tab = reinterpret_cast<float*>(cur);
    cur += tc_table_bytes(s);
    uint8_t* wimg = cur;
    cur += align256((size_t)p.n_otiles * p.n_quads * EDGE_W_SLOT);
    float* partial = reinterpret_cast<float*>(cur);

    cudaError_t e = tc_build_table(grid, tab, s, st);
    if (e != cudaSuccess) return e;
    {
        const int64_t chunks = (int64_t)p.n_otiles * p.n_quads * EDGE_OT * 8;
        int blocks = (int)((chunks + 255) / 256 < (int64_t)sm_count() * 16 ? (chunks + 255) / 256
                                                                            : (int64_t)sm_count() * 16);
        pack_edge_weights_kernel<<<blocks, 256, 0, st>>>(W, bw, nullptr, 1.0f, wimg, s.O, s.I, s.R(), p.n_quads,
                                                         p.n_otiles);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    const int vec_x = ((s.I & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int64_t items = p.n_items();
    const int blocks = (int)(items < sm_count() ? items : sm_count());
    if (split_terms == 3) {
        e = ensure_dynamic_smem<tc_edge_fwd_kernel<3>>((int)EDGE_SMEM_BYTES);
        if (e == cudaSuccess)
            tc_edge_fwd_kernel<3><<<blocks, EDGE_THREADS, EDGE_SMEM_BYTES, st>>>(
                x, s_val, tab, wimg, partial, status, s.N, s.I, s.O, bw ? 1 : 0, p, ti, vec_x);
    } else {
        e = ensure_dynamic_smem<tc_edge_fwd_kernel<1>>((int)EDGE_SMEM_BYTES);
        if (e == cudaSuccess)
            tc_edge_fwd_kernel<1><<<blocks, EDGE_THREADS, EDGE_SMEM_BYTES, st>>>(
                x, s_val, tab, wimg, partial, status, s.N, s.I, s.O, bw ? 1 : 0, p, ti, vec_x);
    }
    if (e != cudaSuccess) return e;
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    const int64_t elems = (int64_t)s.O * s.I;
    int rblocks = (int)((elems + 255) / 256 < (int64_t)sm_count() * 8 ? (elems + 255) / 256 : (int64_t)sm_count() * 8);
    edge_sum_slabs_kernel<<<rblocks, 256, 0, st>>>(partial, a, elems, p.n_slabs(), 1.0f / (float)s.N);
    return cudaGetLastError();
}

// Backward on the tensor cores: float32, G + k <= 8, up to 256 outputs, SiLU (or no) base branch.
bool tc_edge_bwd_supported(const LayerShape& s) {
    return tc_edge_supported(s) && s.O <= EDGE_OT * EDGE_MAX_OTILES && s.N >= 1;
}

size_t tc_edge_bwd_workspace(const LayerShape& s, bool need_x) {
    const EdgeBwdPlan p = plan_edge_bwd(s.N, s.I, s.O);
    const size_t img = align256((size_t)p.n_otiles * p.n_quads * EDGE_W_SLOT);
    return kWsHeader + tc_table_bytes(s) + img * (need_x ? 2 : 1) +
           align256((size_t)p.splits * s.O * s.I * 9 * sizeof(float));
}

// ga = gradient of the loss with respect to a [O, I]; W the effective coefficients; gx, dbw, dW may be NULL.
cudaError_t tc_edge_backward(const float* ga, const float* x, const float* grid, const float* bw, const float* W,
                             float* gx, float* dbw, float* dW, const LayerShape& s, void* ws, size_t ws_bytes,
                             cudaStream_t st) {
    const bool need_x = gx != nullptr;
    if (!ws || ws_bytes < tc_edge_bwd_workspace(s, need_x)) return cudaErrorMemoryAllocation;
    const EdgeBwdPlan p = plan_edge_bwd(s.N, s.I, s.O);
    const TabInfo ti = make_tab_info(s.G, s.K);
    int* status = reinterpret_cast<int*>(ws);
    uint8_t* cur = reinterpret_cast<uint8_t*>(ws) + kWsHeader;
    float* tab = reinterpret_cast<float*>(cur);
    cur += tc_table_bytes(s);
    const size_t img = align256((size_t)p.n_otiles * p.n_quads * EDGE_W_SLOT);
    uint8_t* wimg = cur;
    cur += img;
    uint8_t* wgimg = need_x ? cur : nullptr;
    if (need_x) cur += img;
    float* slabs = reinterpret_cast<float*>(cur);

    cudaError_t e = tc_build_table(grid, tab, s, st);
    if (e != cudaSuccess) return e;
    const int64_t chunks = (int64_t)p.n_otiles * p.n_quads * EDGE_OT * EDGE_FQ;
    const int pblocks = (int)((chunks + 255) / 256 < (int64_t)sm_count() * 16 ? (chunks + 255) / 256
                                                                              : (int64_t)sm_count() * 16);
    pack_edge_weights_pairs_kernel<<<pblocks, 256, 0, st>>>(W, bw, nullptr, 1.0f, wimg, s.O, s.I, s.R(), p.n_quads,
                                                            p.n_otiles);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (need_x) {
        pack_edge_weights_pairs_kernel<<<pblocks, 256, 0, st>>>(W, bw, ga, 1.0f / (float)s.N, wgimg, s.O, s.I, s.R(),
                                                                p.n_quads, p.n_otiles);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (need_x && p.n_otiles > 1) {
        e = cudaMemsetAsync(gx, 0, (size_t)s.N * s.I * sizeof(float), st);
        if (e != cudaSuccess) return e;
    }
    const int vec_x = ((s.I & 1) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      (!gx || (reinterpret_cast<uintptr_t>(gx) & 15) == 0);
    const int64_t items = p.n_items();
    const int blocks = (int)(items < sm_count() ? items : sm_count());
    e = ensure_dynamic_smem<tc_edge_bwd_kernel>((int)EB_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    tc_edge_bwd_kernel<<<blocks, EB_THREADS, EB_SMEM_BYTES, st>>>(x, tab, wimg, wgimg, ga, W, bw, slabs, gx, status, s.N,
                                                                  s.I, s.O, s.R(), p, ti, vec_x, g_sign_recheck ? 1 : 0);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (dW || (dbw && bw)) {
        const int64_t total = (int64_t)s.O * s.I * 9;
        const int fblocks = (int)((total + 255) / 256 < (int64_t)sm_count() * 8 ? (total + 255) / 256
                                                                                : (int64_t)sm_count() * 8);
        edge_bwd_finalize_kernel<<<fblocks, 256, 0, st>>>(slabs, p.splits, W, bw, dW, bw ? dbw : nullptr, (int64_t)s.O * s.I,
                                                          s.R());
        e = cudaGetLastError();
    }
    return e;
}

void tc_edge_set_sign_recheck(bool on) { g_sign_recheck = on; }
bool tc_edge_get_sign_recheck() { return g_sign_recheck; }

}  // namespace kanb200
