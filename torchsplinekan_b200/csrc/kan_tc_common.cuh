// Building blocks shared by the tensor-core kernels (kan_tc.cu: layer forward / backward;
// kan_tc_edge.cu: edge statistic): tile constants, the geometry of the per-span polynomial table,
// the operand producers (window evaluation, placement into 16-byte column chunks, SiLU chunks).
#pragma once
#include "kan_internal.h"
#include "kan_table.cuh"
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
// Per-span polynomial table.
//
// On a knot span [t_m, t_{m+1}) each of the k+1 non-zero basis functions is a
// polynomial of degree k in u = x - t_m.  A small kernel expands the de Boor
// recurrence symbolically (in double) once per call and stores, per feature, a header
// (flag "knots differ from feature 0", the knots) and one 20-float entry per span:
//       16 coefficients c[j][p] (function j of the window, power p of u),
//       t_m, the window start s = m - k (as int bits), 2 unused;
//       coefficients of window slots outside [0, R) are zero, and the entry after the last
//       span is all zero -- it is the one inputs outside the knot range select.
// (TabInfo below gives the offsets.)
// The operand producers then need one span search (compare-and-count up to 12 knots, a
// branch-free binary search beyond), five 16-byte loads and a Horner evaluation per input; the same code serves uniform
// and non-uniform knots.  Conventions (half-open spans, last span closed,
// zero-length spans contribute zero) are those of the dense recurrence.
// ---------------------------------------------------------------------------
constexpr int TAB_FAST_MAX_KNOTS = 12;        // compare-and-count span search up to this many knots
constexpr int TAB_SMEM_FLOATS = 256;          // table of one feature with <= 12 knots: 16 + 12 * 20

// Geometry of the table and of the column space, passed to every kernel.
//   feature block : [0] "differs from feature 0" flag, [1,4) unused,
//                   nk <= 12 : [4,15) knots t_0..t_{nk-2} padded with +inf, [15] = t_{nk-1}
//                   nk  > 12 : [4, 4+nk) the raw knots
//                   [es + 20 e, es + 20 e + 20), e = 0..nk-1 : entry of span e; entry nk-1 is all
//                   zero and is the one inputs outside the knot range select
//   column space  : a feature owns cpf = ceil(R / 8) chunks of 8 slots; chunk g = f * cpf + cw
//                   holds slots 8 cw .. 8 cw + 7 (slots >= R are zero)
struct TabInfo {
    int nk;        // knots per feature
    int es;        // offset of the first entry within a feature block
    int fs;        // floats per feature block
    int cpf;       // chunks of 8 column slots per feature
};

inline TabInfo make_tab_info(int G, int K) {
    TabInfo t;
    t.nk = G + 2 * K + 1;
    t.es = t.nk <= TAB_FAST_MAX_KNOTS ? 16 : ((4 + t.nk + 3) / 4) * 4;
    t.fs = t.es + TAB_ENTRY_FLOATS * t.nk;
    t.cpf = (G + K + 7) / 8;
    return t;
}

// True when every feature has the knot row of feature 0 (the default uniform grid): the kernels
// then keep that single 1-KB table in shared memory instead of reading per-feature tables through
// L1.  Block-wide vote over the per-feature flags the table kernel left in slot 0; every thread
// of the CTA must call it.
__device__ __forceinline__ bool grid_is_shared(const float* __restrict__ tab, int I, const TabInfo& ti) {
    int differs = ti.nk > TAB_FAST_MAX_KNOTS ? 1 : 0;      // only the small table fits in shared memory
    for (int f = threadIdx.x; f < I; f += blockDim.x)
        if (__ldg(tab + (size_t)f * ti.fs) != 0.0f) differs = 1;
    return __syncthreads_or(differs) == 0;
}

// Index of the table entry of x: the knot span (last knot <= x; the last span is closed on the
// right), or the all-zero entry nk - 1 for x outside the knot range / NaN.
// WIDE = false promises at most 12 knots (G + k <= 8).
template <bool SMEM_TAB, bool WIDE>
__device__ __forceinline__ int table_entry_index(const float* __restrict__ ftab, const TabInfo& ti, float xv) {
    auto ld4 = [](const float4* p) -> float4 { return SMEM_TAB ? *p : __ldg(p); };
    if (!WIDE || ti.nk <= TAB_FAST_MAX_KNOTS) {
        const float4 k0 = ld4(reinterpret_cast<const float4*>(ftab + 4));
        const float4 k1 = ld4(reinterpret_cast<const float4*>(ftab + 4) + 1);
        const float4 k2 = ld4(reinterpret_cast<const float4*>(ftab + 4) + 2);
        return entry_index12(k0, k1, k2, ti.nk, xv);
    }
    const float* t = ftab + 4;
    const float t_last = SMEM_TAB ? t[ti.nk - 1] : __ldg(t + ti.nk - 1);
    const float t_first = SMEM_TAB ? t[0] : __ldg(t);
    const bool inside = (xv >= t_first) && (xv <= t_last);
    int lo = 0, hi = ti.nk - 1;                // t[lo] <= x < t[hi] while inside and x < t_last
#pragma unroll
    for (int it = 0; it < 7; ++it) {           // 2^7 > 72 knots
        const int mid = (lo + hi) >> 1;
        const float tm = SMEM_TAB ? t[mid] : __ldg(t + mid);
        const bool open = (hi - lo) > 1;
        const bool right = tm <= xv;
        lo = (open && right) ? mid : lo;
        hi = (open && !right) ? mid : hi;
    }
    const int m = (xv == t_last) ? ti.nk - 2 : lo;
    return inside ? m : ti.nk - 1;
}

__device__ __forceinline__ float silu_fast(float x) {
    return __fdividef(x, 1.0f + __expf(-x));
}

// The k + 1 non-zero basis values of one input (packed as bf16 pairs, hi and lo parts) and the
// column slot s of the first one.  Inputs outside the knot range select the all-zero entry.
struct Window {
    uint32_t h01, h23, l01, l23;
    int s;
};

template <bool SPLIT, bool SMEM_TAB, bool WIDE>
__device__ __forceinline__ Window eval_window(const float* __restrict__ ftab, const TabInfo& ti, float xv) {
    auto ld4 = [](const float4* p) -> float4 { return SMEM_TAB ? *p : __ldg(p); };
    const int m = table_entry_index<SMEM_TAB, WIDE>(ftab, ti, xv);
    const float4* ent = reinterpret_cast<const float4*>(ftab + ti.es + m * TAB_ENTRY_FLOATS);
    const float4 c0 = ld4(ent), c1 = ld4(ent + 1), c2 = ld4(ent + 2), c3 = ld4(ent + 3), meta = ld4(ent + 4);
    const float u = xv - meta.x;
    const float v0 = fmaf(fmaf(fmaf(c0.w, u, c0.z), u, c0.y), u, c0.x);
    const float v1 = fmaf(fmaf(fmaf(c1.w, u, c1.z), u, c1.y), u, c1.x);
    const float v2 = fmaf(fmaf(fmaf(c2.w, u, c2.z), u, c2.y), u, c2.x);
    const float v3 = fmaf(fmaf(fmaf(c3.w, u, c3.z), u, c3.y), u, c3.x);
    Window w;
    w.s = __float_as_int(meta.y);
    w.l01 = 0;
    w.l23 = 0;
    if (SPLIT) {
        split2(v0, v1, w.h01, w.l01);
        split2(v2, v3, w.h23, w.l23);
    } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v0, v1);
        const __nv_bfloat162 b = __floats2bfloat162_rn(v2, v3);
        w.h01 = *reinterpret_cast<const uint32_t*>(&a);
        w.h23 = *reinterpret_cast<const uint32_t*>(&b);
    }
    return w;
}

// Chunk `cw` of the feature's column slots (slots 8 cw .. 8 cw + 7) as two 128-bit rows (hi and
// lo bf16 parts): the 4 half-words of the window go to half-word offset s - 8 cw; a window that
// does not touch the chunk leaves zeros.  Branch-free.  SPLIT = false leaves lo untouched.
template <bool SPLIT>
__device__ __forceinline__ void place_window(const Window& w, int cw, uint4& hi, uint4& lo) {
    const int s = w.s - 8 * cw;
    // With s = 2 q + odd the payload becomes three words (t0, t1, t2) that start at word q.
    const int odd = s & 1;
    const int q = (s - odd) >> 1;                          // -2 .. 3 when the window touches the chunk
    const bool at0 = (q == 0), at1 = (q == 1), at2 = (q == 2), at3 = (q == 3), atm1 = (q == -1), atm2 = (q == -2);
    auto place = [&](uint32_t w01, uint32_t w23) -> uint4 {
        const uint32_t t0 = odd ? (w01 << 16) : w01;
        const uint32_t t1 = odd ? __funnelshift_r(w01, w23, 16) : w23;
        const uint32_t t2 = odd ? (w23 >> 16) : 0u;
        uint4 o;
        o.x = at0 ? t0 : (atm1 ? t1 : (atm2 ? t2 : 0u));
        o.y = at1 ? t0 : (at0 ? t1 : (atm1 ? t2 : 0u));
        o.z = at2 ? t0 : (at1 ? t1 : (at0 ? t2 : 0u));
        o.w = at3 ? t0 : (at2 ? t1 : (at1 ? t2 : 0u));
        return o;
    };
    hi = place(w.h01, w.h23);
    if (SPLIT) lo = place(w.l01, w.l23);
}

// Derivatives of the window functions of one input from its feature's table:
// d/du (c0 + c1 u + c2 u^2 + c3 u^3) = c1 + 2 c2 u + 3 c3 u^2.  Returns the window start; inputs
// outside the knot range select the all-zero entry.
template <bool SMEM_TAB, bool WIDE>
__device__ __forceinline__ int eval_feature_deriv(const float* __restrict__ ftab, const TabInfo& ti, float xv,
                                                  float (&d)[4]) {
    auto ld4 = [](const float4* p) -> float4 { return SMEM_TAB ? *p : __ldg(p); };
    const int m = table_entry_index<SMEM_TAB, WIDE>(ftab, ti, xv);
    const float4* ent = reinterpret_cast<const float4*>(ftab + ti.es + m * TAB_ENTRY_FLOATS);
    const float4 c0 = ld4(ent), c1 = ld4(ent + 1), c2 = ld4(ent + 2), c3 = ld4(ent + 3), meta = ld4(ent + 4);
    const float u = xv - meta.x;
    d[0] = fmaf(fmaf(3.0f * c0.w, u, 2.0f * c0.z), u, c0.y);
    d[1] = fmaf(fmaf(3.0f * c1.w, u, 2.0f * c1.z), u, c1.y);
    d[2] = fmaf(fmaf(3.0f * c2.w, u, 2.0f * c2.z), u, c2.y);
    d[3] = fmaf(fmaf(3.0f * c3.w, u, 2.0f * c3.z), u, c3.y);
    return __float_as_int(meta.y);
}

// Values of the window functions of one input in float32 (no bf16 split); returns the window start.
template <bool SMEM_TAB, bool WIDE>
__device__ __forceinline__ int eval_feature_values(const float* __restrict__ ftab, const TabInfo& ti, float xv,
                                                   float (&v)[4]) {
    auto ld4 = [](const float4* p) -> float4 { return SMEM_TAB ? *p : __ldg(p); };
    const int m = table_entry_index<SMEM_TAB, WIDE>(ftab, ti, xv);
    const float4* ent = reinterpret_cast<const float4*>(ftab + ti.es + m * TAB_ENTRY_FLOATS);
    const float4 c0 = ld4(ent), c1 = ld4(ent + 1), c2 = ld4(ent + 2), c3 = ld4(ent + 3), meta = ld4(ent + 4);
    const float u = xv - meta.x;
    v[0] = fmaf(fmaf(fmaf(c0.w, u, c0.z), u, c0.y), u, c0.x);
    v[1] = fmaf(fmaf(fmaf(c1.w, u, c1.z), u, c1.y), u, c1.x);
    v[2] = fmaf(fmaf(fmaf(c2.w, u, c2.z), u, c2.y), u, c2.x);
    v[3] = fmaf(fmaf(fmaf(c3.w, u, c3.z), u, c3.y), u, c3.x);
    return __float_as_int(meta.y);
}

// sigma(x) (1 + x (1 - sigma(x)))
__device__ __forceinline__ float silu_grad_fast(float x) {
    const float sg = __fdividef(1.0f, 1.0f + __expf(-x));
    return sg * fmaf(x, 1.0f - sg, 1.0f);
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

// Records that a bounded wait ran out (or that the kernel could not start): the workspace's status
// word takes the code if it is still 0 (it is sticky), and when the caller stored a pointer at byte
// 8 of the workspace header -- an int the host can read without synchronising, e.g. in mapped
// pinned memory -- that int receives the code too.
__device__ __forceinline__ void report_status(int* status, int code) {
    atomicCAS(status, 0, code);
    int* mirror = *reinterpret_cast<int* volatile*>(status + 2);
    if (mirror != nullptr) {
        *reinterpret_cast<volatile int*>(mirror) = code;
        __threadfence_system();
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

inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Opt-in to more than 48 KB of dynamic shared memory, once per kernel and device.
template <auto Kernel>
cudaError_t ensure_dynamic_smem(int bytes) {
    static bool done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    return e;
}

}  // namespace
}  // namespace kanb200
