// Parameter-gradient kernel, second formulation (included by kan_tc.cu inside its namespaces):
//
//   D^T[c, o] = sum_n A[n, c] dY[n, o]        M = 128 columns,  N = 2 x 256 outputs,  K = samples
//
// The generated operand (basis windows / SiLU of x) is the M side: 128 columns x 64 samples per
// block of samples feed both 256-output accumulators, so the worker warps produce half as many
// values per tensor-core flop as with the generated operand on the N side.  Both operands are
// MN-major; the dY tiles come from the same image as before (two 16-KB pieces per 32-KB slot).
// Work item = (split of the samples, tile of 128 columns, pair of 256-output tiles).  Every
// `chunk_kb` blocks of 64 samples the accumulator is added into the item's slab of partial sums.
// The two accumulators end their chunks half a chunk apart: while the workers drain one, the MMA
// thread runs up to two blocks ahead on the other (three stages of the generated operand), so
// the tensor pipe keeps working during most of a drain.
constexpr int B2_G_STAGES = 3, B2_B_SLOTS = 4;
constexpr uint32_t B2_G_STAGE_BYTES = 2 * TILE_A_BYTES;                  // hi + lo, 128 c x 64 n
constexpr uint32_t B2_SMEM_G = 0;
constexpr uint32_t B2_SMEM_B = B2_SMEM_G + B2_G_STAGES * B2_G_STAGE_BYTES;
constexpr uint32_t B2_SMEM_CTRL = B2_SMEM_B + B2_B_SLOTS * TILE_B_BYTES;
constexpr uint32_t B2_CTRL_BYTES = 256 + TAB_SMEM_FLOATS * 4;            // barriers + the shared-grid table
constexpr uint32_t B2_SMEM_BYTES = B2_SMEM_CTRL + B2_CTRL_BYTES;
static_assert(B2_SMEM_BYTES <= 232448, "backward kernel shared memory exceeds 227 KB");
constexpr int B2_LOOKAHEAD = B2_G_STAGES - 1;      // blocks one accumulator may run ahead of the other

struct B2Ctrl {
    uint64_t fullG[B2_G_STAGES], emptyG[B2_G_STAGES];
    uint64_t fullB[B2_B_SLOTS], emptyB[B2_B_SLOTS];
    uint64_t chunkFull[2], drained[2];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(B2Ctrl) <= 256, "control block too large");

struct Bwd2Plan {
    int n_otiles;          // tiles of 256 outputs (the dY image has two 128-output groups per tile)
    int n_opairs;          // pairs of such tiles: the two accumulators of an item
    int ct_spline;         // column tiles of 16 chunks (8 slots each) of the spline part
    int ct_base;           // column tiles of 128 base features
    int splits;
    int chunk_kb;          // 64-sample blocks accumulated in TMEM between drains (even)
    int64_t kb_total;      // 64-sample blocks
    int64_t kb_per_split;
    __host__ __device__ int n_ctiles() const { return ct_spline + ct_base; }
    __host__ __device__ int64_t n_items() const { return (int64_t)n_opairs * n_ctiles() * splits; }
    // floats of one split's slab: every (o-pair, c-tile) owns a 128 x 512 block
    __host__ __device__ int64_t slab_floats() const { return (int64_t)n_opairs * n_ctiles() * 128 * 512; }
};

// The order in which the MMA thread and the dY copy thread walk the (block of samples, accumulator)
// pairs of one item.  Blocks are visited in order, accumulator 0 before 1, except after a chunk of
// accumulator h has ended at block t - 1: then the other accumulator first takes blocks
// t .. t + la (la <= B2_LOOKAHEAD) and h follows with the same blocks, which gives the workers the
// time of la + 1 half-blocks to drain h.  Chunks of accumulator 0 start at multiples of `chunk`,
// those of accumulator 1 half a chunk later (its first chunk is short).
struct B2Schedule {
    int K, nsub, chunk;
    int k;            // first block of the current group
    int la;           // the group covers blocks k .. k + la
    int first;        // accumulator that goes first in the group
    int pos;          // position within the group: 0 .. nsub * (la + 1) - 1
    __device__ void init(int K_, int nsub_, int chunk_) {
        K = K_; nsub = nsub_; chunk = chunk_;
        k = 0;
        start_group();
    }
    __device__ bool boundary(int h, int kk) const {          // does a chunk of accumulator h start at kk?
        if (kk <= 0) return false;
        return h == 0 ? (kk % chunk) == 0 : (kk % chunk) == chunk / 2;
    }
    __device__ void start_group() {
        pos = 0;
        la = 0;
        first = 0;
        if (nsub == 2 && k < K) {
            const int h = boundary(0, k) ? 0 : (boundary(1, k) ? 1 : -1);
            if (h >= 0) {
                first = 1 - h;
                la = (K - 1 - k < B2_LOOKAHEAD) ? K - 1 - k : B2_LOOKAHEAD;
            }
        }
    }
    __device__ bool done() const { return k >= K; }
    __device__ void current(int& kk, int& h) const {
        const int per = la + 1;
        h = (nsub == 1) ? 0 : ((pos < per) ? first : 1 - first);
        kk = k + (pos % per);
    }
    __device__ void advance() {
        ++pos;
        if (pos >= nsub * (la + 1)) {
            k += la + 1;
            start_group();
        }
    }
    // chunk bookkeeping of accumulator h at block kk
    __device__ bool chunk_starts(int h, int kk) const { return kk == 0 || boundary(h, kk); }
    __device__ bool chunk_ends(int h, int kk) const { return kk == K - 1 || boundary(h, kk + 1); }
};

template <int NTERMS, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_bwd_param2_kernel(const float* __restrict__ x, const float* __restrict__ tab, const uint8_t* __restrict__ dyimg,
                     float* __restrict__ partial, int* __restrict__ status,
                     int64_t N, int I, int O, Bwd2Plan plan, TabInfo ti, int vec_ok) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr bool SPLIT = (NTERMS == 3);
    const uint32_t sbase = smem_u32(smem);
    B2Ctrl* ctrl = reinterpret_cast<B2Ctrl*>(smem + B2_SMEM_CTRL);
    float* stab = reinterpret_cast<float*>(smem + B2_SMEM_CTRL + 256);
    volatile int* abort_flag = &ctrl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool shared_grid = grid_is_shared(tab, I, ti);
    if (shared_grid && threadIdx.x < TAB_SMEM_FLOATS && threadIdx.x < ti.fs) stab[threadIdx.x] = tab[threadIdx.x];
    const int n_ohalves = plan.n_otiles * 2;
    const int n_ctiles = plan.n_ctiles();
    const int64_t n_items = plan.n_items();

    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, kStatusBadSmem);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < B2_G_STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->fullG[s]), WORKER_THREADS);
            mbar_init(smem_u32(&ctrl->emptyG[s]), 1);
        }
        for (int s = 0; s < B2_B_SLOTS; ++s) {
            mbar_init(smem_u32(&ctrl->fullB[s]), 1);
            mbar_init(smem_u32(&ctrl->emptyB[s]), 1);
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

    // item -> (split, o-pair, c-tile); consecutive items share the o-pair (same dY tiles in L2).
    auto decode = [&](int64_t item, int& sp, int& op, int& ct) {
        ct = (int)(item % n_ctiles);
        const int64_t rest = item / n_ctiles;
        op = (int)(rest % plan.n_opairs);
        sp = (int)(rest / plan.n_opairs);
    };
    auto k_range = [&](int sp, int64_t& kb0, int64_t& kb1) {
        kb0 = (int64_t)sp * plan.kb_per_split;
        kb1 = kb0 + plan.kb_per_split;
        if (kb1 > plan.kb_total) kb1 = plan.kb_total;
    };
    auto n_sub = [&](int op) -> int { return (plan.n_otiles - 2 * op) >= 2 ? 2 : 1; };

    if (warp < WORKER_WARPS) {
        // ===== workers: 64 samples x 128 columns per block, MN-major; drains in between =====
        const int quad = warp & 3, part = warp >> 2;
        const int n_loc = (warp & 1) * 32 + lane;       // sample within the block
        const int cp = warp >> 1;                       // pair of chunks 2 cp, 2 cp + 1 of the tile
        const int kk = n_loc & 7;
        uint32_t it = 0;                                // generated tiles so far (stage ring)
        uint32_t n_drained[2] = {0, 0};
        bool ok = true;

        // adds (or stores, for the first chunk of the item) accumulator h into the item's slab
        auto drain = [&](int h, int sp, int op, int ct, bool first) -> bool {
            if (!mbar_wait(smem_u32(&ctrl->chunkFull[h]), n_drained[h] & 1u, abort_flag)) return false;
            ++n_drained[h];
            tc_fence_after_sync();
            // blocked layout: tile (split, o-pair, c-tile) -> [output / 4][column row][4 floats]
            float4* tile = reinterpret_cast<float4*>(partial) +
                           (((size_t)sp * plan.n_opairs + op) * n_ctiles + ct) * (size_t)(128 * 128);
            const int row = quad * 32 + lane;
#pragma unroll 1
            for (int c = part; c < BLOCK_N / 32; c += 4) {
                float4* dst = tile + ((size_t)(h * 64 + c * 8)) * 128 + row;
                float4 old[8];
                if (!first) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) old[q] = dst[(size_t)q * 128];
                }
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + h * BLOCK_N + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                           __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                    if (!first) {
                        v.x += old[q].x; v.y += old[q].y; v.z += old[q].z; v.w += old[q].w;
                    }
                    dst[(size_t)q * 128] = v;
                }
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctrl->drained[h]));
            return true;
        };

        for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int sp, op, ct;
            decode(item, sp, op, ct);
            const bool spline = ct < plan.ct_spline;
            const int nsub = n_sub(op);
            int64_t kb0, kb1;
            k_range(sp, kb0, kb1);
            const int K = (int)(kb1 - kb0);
            B2Schedule sch;
            sch.init(K, nsub, plan.chunk_kb);
            // the thread's two chunks: g = 16 ct + 2 cp + q belongs to feature g / cpf, slots 8 (g % cpf) ..
            int cf[2], ccw[2];
            {
                const int g0 = ct * 16 + cp * 2;
                const int cpf = WIDE ? ti.cpf : 1;
                cf[0] = g0 / cpf;
                ccw[0] = g0 - cf[0] * cpf;
                cf[1] = cf[0];
                ccw[1] = ccw[0] + 1;
                if (ccw[1] == cpf) { cf[1] += 1; ccw[1] = 0; }
            }
            const int fb0 = (ct - plan.ct_spline) * 128 + cp * 16;      // base tiles: first of 16 features
            float nx[2] = {0.f, 0.f};
            auto prefetch_spline = [&](int64_t kb) {
                const int64_t n = kb * BLOCK_K + n_loc;
                nx[0] = nx[1] = 0.f;
                if (n < N) {
                    const float* xr = x + (size_t)n * I;
                    if (cf[0] < I) nx[0] = __ldg(xr + cf[0]);
                    if (cf[1] < I) nx[1] = (cf[1] == cf[0]) ? nx[0] : __ldg(xr + cf[1]);
                }
            };
            if (spline) prefetch_spline(kb0);
            bool first_drain[2] = {true, true};
            // per accumulator: the block after whose production its finished chunk is drained (-1: none)
            int pend_at[2] = {-1, -1};
            for (int kl = 0; kl < K; ++kl, ++it) {
                const int64_t kb = kb0 + kl;
                const uint32_t stage = it % B2_G_STAGES;
                const uint32_t g_hi = sbase + B2_SMEM_G + stage * B2_G_STAGE_BYTES;
                const uint32_t g_lo = g_hi + TILE_A_BYTES;
                const bool n_ok = kb * BLOCK_K + n_loc < N;
                if (spline) {
                    const float xv0 = nx[0], xv1 = nx[1];
                    if (kl + 1 < K) prefetch_spline(kb + 1);
                    if (!mbar_wait(smem_u32(&ctrl->emptyG[stage]), ((it / B2_G_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    Window w;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int f = cf[q];
                        if (!WIDE || q == 0 || f != cf[0]) {                 // uniform over the warp
                            const float xv = q == 0 ? xv0 : xv1;
                            if (shared_grid)
                                w = eval_window<SPLIT, true, WIDE>(stab, ti, xv);
                            else
                                w = eval_window<SPLIT, false, WIDE>(tab + (size_t)(f < I ? f : I - 1) * ti.fs, ti, xv);
                        }
                        uint4 hi, lo;
                        place_window<SPLIT>(w, ccw[q], hi, lo);
                        if (!(n_ok && f < I)) {
                            hi = make_uint4(0, 0, 0, 0);
                            lo = hi;
                        }
                        const int fl = cp * 2 + q;                           // chunk within the tile, 0..15
                        const uint32_t off = (uint32_t)((fl >> 3) * 8 + (n_loc >> 3)) * 1024u + (uint32_t)kk * 128u +
                                             (uint32_t)(((fl & 7) ^ kk) << 4);
                        st_shared_v4(g_hi + off, hi);
                        if (SPLIT) st_shared_v4(g_lo + off, lo);
                    }
                } else {
                    float xv[2][8];
                    const int64_t n = kb * BLOCK_K + n_loc;
                    load_x8(x, n, n_ok, I, fb0, vec_ok != 0, xv[0]);
                    load_x8(x, n, n_ok, I, fb0 + 8, vec_ok != 0, xv[1]);
                    if (!mbar_wait(smem_u32(&ctrl->emptyG[stage]), ((it / B2_G_STAGES) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        uint4 hi, lo;
                        silu_chunk<SPLIT>(xv[q], hi, lo);
                        const int fl = cp * 2 + q;
                        const uint32_t off = (uint32_t)((fl >> 3) * 8 + (n_loc >> 3)) * 1024u + (uint32_t)kk * 128u +
                                             (uint32_t)(((fl & 7) ^ kk) << 4);
                        st_shared_v4(g_hi + off, hi);
                        if (SPLIT) st_shared_v4(g_lo + off, lo);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ctrl->fullG[stage]));

                // A chunk that ends with this block is drained once the blocks the other accumulator
                // may run ahead on have been produced, so that the tensor pipe has work meanwhile.
                // Pass 0: drains that are due; pass 1: chunks ending now are registered (an older
                // chunk of the same accumulator goes first); pass 2: those due at once (item end).
#pragma unroll 1
                for (int pass = 0; pass < 3 && ok; ++pass) {
#pragma unroll 1
                    for (int h = 0; h < nsub && ok; ++h) {
                        const bool reg = (pass == 1) && sch.chunk_ends(h, kl);
                        const bool due = pend_at[h] >= 0 && (pass == 1 ? reg : kl >= pend_at[h]);
                        if (due) {
                            ok = drain(h, sp, op, ct, first_drain[h]);
                            first_drain[h] = false;
                            pend_at[h] = -1;
                        }
                        if (reg) {
                            int at = kl + 1 + (nsub == 2 ? B2_LOOKAHEAD : 0);
                            pend_at[h] = at > K - 1 ? K - 1 : at;
                        }
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(BLOCK_N, true, true);
            constexpr uint64_t dbase = make_sdesc_sw128(8192, 1024);
            uint32_t it0 = 0, bslot = 0;
            uint32_t n_chunks[2] = {0, 0};
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int sp, op, ct;
                decode(item, sp, op, ct);
                const int nsub = n_sub(op);
                int64_t kb0, kb1;
                k_range(sp, kb0, kb1);
                const int K = (int)(kb1 - kb0);
                B2Schedule sch;
                sch.init(K, nsub, plan.chunk_kb);
                for (; !sch.done() && ok; sch.advance()) {
                    int kl, h;
                    sch.current(kl, h);
                    const uint32_t it = it0 + (uint32_t)kl;
                    const uint32_t stage = it % B2_G_STAGES;
                    const uint32_t g_hi = sbase + B2_SMEM_G + stage * B2_G_STAGE_BYTES;
                    const uint32_t g_lo = g_hi + TILE_A_BYTES;
                    const bool chunk_start = sch.chunk_starts(h, kl);
                    if (chunk_start && n_chunks[h] > 0) {
                        // the accumulator may be overwritten only after the workers have drained it
                        if (!mbar_wait(smem_u32(&ctrl->drained[h]), (n_chunks[h] - 1) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                    }
                    if (!mbar_wait(smem_u32(&ctrl->fullG[stage]), (it / B2_G_STAGES) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + h * BLOCK_N;
                    const uint32_t slot_h = bslot % B2_B_SLOTS;
                    if (!mbar_wait(smem_u32(&ctrl->fullB[slot_h]), (bslot / B2_B_SLOTS) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t b_hi = sbase + B2_SMEM_B + slot_h * TILE_B_BYTES;
#pragma unroll
                    for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                        mma_f16_ss(d_tmem, sdesc_at(dbase, g_hi + ks * 2048), sdesc_at(dbase, b_hi + ks * 2048),
                                   idesc, (!chunk_start || ks > 0) ? 1u : 0u);
                    if (SPLIT) {
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, g_lo + ks * 2048), sdesc_at(dbase, b_hi + ks * 2048),
                                       idesc, 1u);
                    }
                    mma_commit(smem_u32(&ctrl->emptyB[slot_h]));
                    ++bslot;
                    if (SPLIT) {
                        const uint32_t slot_l = bslot % B2_B_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->fullB[slot_l]), (bslot / B2_B_SLOTS) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t b_lo = sbase + B2_SMEM_B + slot_l * TILE_B_BYTES;
#pragma unroll
                        for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks)
                            mma_f16_ss(d_tmem, sdesc_at(dbase, g_hi + ks * 2048), sdesc_at(dbase, b_lo + ks * 2048),
                                       idesc, 1u);
                        mma_commit(smem_u32(&ctrl->emptyB[slot_l]));
                        ++bslot;
                    }
                    // the stage is free once the accumulator that comes second in the group has used it
                    if (nsub == 1 || h == 1 - sch.first) mma_commit(smem_u32(&ctrl->emptyG[stage]));
                    if (sch.chunk_ends(h, kl)) {
                        mma_commit(smem_u32(&ctrl->chunkFull[h]));
                        ++n_chunks[h];
                    }
                }
                it0 += (uint32_t)K;
            }
        }
    } else {
        if (lane == 0) {
            // ===== bulk copies of the dY tiles, in the order the MMA thread uses them =====
            uint32_t bslot = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int sp, op, ct;
                decode(item, sp, op, ct);
                const int nsub = n_sub(op);
                int64_t kb0, kb1;
                k_range(sp, kb0, kb1);
                B2Schedule sch;
                sch.init((int)(kb1 - kb0), nsub, plan.chunk_kb);
                for (; !sch.done() && ok; sch.advance()) {
                    int kl, h;
                    sch.current(kl, h);
                    const int64_t kb = kb0 + kl;
                    const int oh0 = 2 * (2 * op + h);                      // first of two 128-output groups
                    for (int term = 0; term < (SPLIT ? 2 : 1); ++term, ++bslot) {
                        const uint32_t slot = bslot % B2_B_SLOTS;
                        if (!mbar_wait(smem_u32(&ctrl->emptyB[slot]), ((bslot / B2_B_SLOTS) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = smem_u32(&ctrl->fullB[slot]);
                        mbar_arrive_expect_tx(bar, TILE_B_BYTES);
                        for (int piece = 0; piece < 2; ++piece) {
                            const uint8_t* src = dyimg + (((size_t)kb * n_ohalves + (size_t)(oh0 + piece)) * 2 + term) *
                                                             (size_t)TILE_A_BYTES;
                            bulk_g2s(sbase + B2_SMEM_B + slot * TILE_B_BYTES + piece * TILE_A_BYTES, src, TILE_A_BYTES,
                                     bar);
                        }
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

// Sums the per-split slabs of tc_bwd_param2_kernel and applies the scaler algebra: gsw = scaler * D,
// gscaler = sum_r sw * D, gbw = base column.  Thread = (feature, group of 4 outputs), feature
// fastest: a thread reads the 8 rows of a chunk as 8 consecutive 16-byte pieces (4 outputs each)
// and consecutive threads read consecutive chunks, so slab reads and parameter writes are both
// contiguous across a warp.
__global__ void __launch_bounds__(256)
finalize2_kernel(const float* __restrict__ partial, Bwd2Plan plan, int cpf,
                 const float* __restrict__ sw, const float* __restrict__ scaler,
                 float* __restrict__ gsw, float* __restrict__ gscaler, float* __restrict__ gbw,
                 int O, int I, int R) {
    const int n_ctiles = plan.n_ctiles();
    const int O4 = (O + 3) / 4;
    const int64_t total = (int64_t)O4 * I;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % I), oq = (int)(idx / I);
        const int o0 = oq * 4;
        const int op = o0 >> 9, oql = (o0 & 511) >> 2;            // pair of 256-output tiles, quad within it
        auto tile_ptr = [&](int sp, int ct) -> const float4* {
            return reinterpret_cast<const float4*>(partial) +
                   (((size_t)sp * plan.n_opairs + op) * n_ctiles + ct) * (size_t)(128 * 128) + (size_t)oql * 128;
        };
        if (gsw || gscaler) {
            float sc[4], gs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[e] = (scaler && o0 + e < O) ? scaler[(size_t)(o0 + e) * I + i] : 1.0f;
            for (int cw = 0; cw < cpf; ++cw) {
                const int g = i * cpf + cw, ct = g >> 4, row0 = (g & 15) * 8;
                float4 v[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp = 0; sp < plan.splits; ++sp) {
                    const float4* t = tile_ptr(sp, ct) + row0;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const float4 a = t[r];
                        v[r].x += a.x; v[r].y += a.y; v[r].z += a.z; v[r].w += a.w;
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (o0 + e >= O) continue;
                    const size_t oi = (size_t)(o0 + e) * I + i;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const int slot = cw * 8 + r;
                        if (slot < R) {
                            const float d = e == 0 ? v[r].x : (e == 1 ? v[r].y : (e == 2 ? v[r].z : v[r].w));
                            if (gsw) gsw[oi * R + slot] = scaler ? sc[e] * d : d;
                            if (gscaler) gs[e] += sw[oi * R + slot] * d;
                        }
                    }
                }
            }
            if (gscaler) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (o0 + e < O) gscaler[(size_t)(o0 + e) * I + i] = gs[e];
            }
        }
        if (gbw) {
            const int ct = plan.ct_spline + (i >> 7), row = i & 127;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp = 0; sp < plan.splits; ++sp) {
                const float4 a = tile_ptr(sp, ct)[row];
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (o0 + 0 < O) gbw[(size_t)(o0 + 0) * I + i] = v.x;
            if (o0 + 1 < O) gbw[(size_t)(o0 + 1) * I + i] = v.y;
            if (o0 + 2 < O) gbw[(size_t)(o0 + 2) * I + i] = v.z;
            if (o0 + 3 < O) gbw[(size_t)(o0 + 3) * I + i] = v.w;
        }
    }
}
