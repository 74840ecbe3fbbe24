// Self-test of the shared-memory operand layouts of tcgen05.mma.  Built into its own small library
// (lib/libkan_b200_selftest.so) that only the test-suite loads; it is not part of the product ABI.
//
// One CTA copies two caller-built byte images (A: 128 x 64 bf16, B: 256 x 64 bf16) into shared
// memory, issues the four K = 16 MMAs of one 64-wide block with the descriptors of the layout the
// caller NAMES -- the same constexpr descriptor builders the production kernels use -- and writes
// the fp32 accumulator D[128, 256] out.  The test builds the images for the K-major and MN-major
// 128-byte-swizzle layouts and checks the product against numpy, so a wrong descriptor shows up
// as a failed small test instead of a wrong large result.  Descriptors are never taken from the
// caller.
#include "kan_dmma.cuh"
#include "kan_tc_ptx.cuh"

#include <cuda_runtime.h>

namespace kanb200 {

namespace {
using namespace ptx;

constexpr int kLayoutKMajor = 0;     // rows x 128 B, K contiguous (forward: generated operand, weight image)
constexpr int kLayoutMnMajor = 1;    // [64-wide MN group][8-row K group][8 rows][128 B] (backward operands)
constexpr uint32_t kABytes = 128 * 64 * 2, kBBytes = 256 * 64 * 2;
constexpr int kSteps = 4, kCols = 256;

__global__ void __launch_bounds__(128, 1)
umma_layout_kernel(const uint8_t* __restrict__ a_img, const uint8_t* __restrict__ b_img, int layout,
                   float* __restrict__ D, int* __restrict__ status) {
    const bool mn = layout == kLayoutMnMajor;
    const uint32_t a_bytes = kABytes, b_bytes = kBBytes;
    const uint64_t a_desc = mn ? make_sdesc_sw128(8192, 1024) : make_sdesc_sw128(16, 1024), b_desc = a_desc;
    const uint32_t idesc = make_idesc_bf16(kCols, mn, mn);
    const uint32_t a_step = mn ? 2048u : 32u, b_step = a_step;
    const int ksteps = kSteps, ncols = kCols;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, 2);
        return;
    }
    const uint32_t a_off = 0, b_off = (a_bytes + 1023u) & ~1023u;
    for (uint32_t e = threadIdx.x * 16; e < a_bytes; e += blockDim.x * 16)
        *reinterpret_cast<uint4*>(smem + a_off + e) = *reinterpret_cast<const uint4*>(a_img + e);
    for (uint32_t e = threadIdx.x * 16; e < b_bytes; e += blockDim.x * 16)
        *reinterpret_cast<uint4*>(smem + b_off + e) = *reinterpret_cast<const uint4*>(b_img + e);
    fence_proxy_async_smem();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        for (int ks = 0; ks < ksteps; ++ks)
            mma_f16_ss(tmem_base, sdesc_at(a_desc, sbase + a_off + ks * a_step),
                       sdesc_at(b_desc, sbase + b_off + ks * b_step), idesc, ks > 0 ? 1u : 0u);
        mma_commit(smem_u32(&done_bar));
    }
    __syncwarp();
    const bool ok = mbar_wait(smem_u32(&done_bar), 0, &abort_flag);
    tc_fence_after_sync();
    if (ok) {
        const int row = warp * 32 + lane;
        for (int c = 0; c < ncols / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + c * 32, r);
            tmem_ld_wait();
            for (int q = 0; q < 32; ++q) D[(size_t)row * ncols + c * 32 + q] = __uint_as_float(r[q]);
        }
    } else {
        if (lane == 0) atomicExch(status, 1);
        __nanosleep(100000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}
// The same with every layout parameter named by the caller (strides in bytes, all fed through the
// production descriptor builder): operands of up to 32 KB each, `ksteps` K = 16 steps, N columns.
// Used to pin down the readings of ONE shared tile by two different products, e.g. a K-major
// [rows][64] tile read as an MN-major operand whose 16 columns start 32 q bytes into every row.
struct GeneralLayout {
    uint32_t a_bytes, b_bytes;
    uint32_t a_mn, b_mn;             // 1 = MN-major
    uint32_t a_lbo, a_sbo, a_step, a_off;
    uint32_t b_lbo, b_sbo, b_step, b_off;
    uint32_t n, ksteps;
};

__global__ void __launch_bounds__(128, 1)
umma_general_kernel(const uint8_t* __restrict__ a_img, const uint8_t* __restrict__ b_img, GeneralLayout L,
                    float* __restrict__ D, int* __restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((sbase & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, 2);
        return;
    }
    const uint32_t a_base = 0, b_base = 32768;
    for (uint32_t e = threadIdx.x * 16; e < L.a_bytes; e += blockDim.x * 16)
        *reinterpret_cast<uint4*>(smem + a_base + e) = *reinterpret_cast<const uint4*>(a_img + e);
    for (uint32_t e = threadIdx.x * 16; e < L.b_bytes; e += blockDim.x * 16)
        *reinterpret_cast<uint4*>(smem + b_base + e) = *reinterpret_cast<const uint4*>(b_img + e);
    fence_proxy_async_smem();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        const uint64_t a_desc = make_sdesc_sw128(L.a_lbo, L.a_sbo), b_desc = make_sdesc_sw128(L.b_lbo, L.b_sbo);
        const uint32_t idesc = make_idesc_bf16((int)L.n, L.a_mn != 0, L.b_mn != 0);
        for (uint32_t ks = 0; ks < L.ksteps; ++ks)
            mma_f16_ss(tmem_base, sdesc_at(a_desc, sbase + a_base + L.a_off + ks * L.a_step),
                       sdesc_at(b_desc, sbase + b_base + L.b_off + ks * L.b_step), idesc, ks > 0 ? 1u : 0u);
        mma_commit(smem_u32(&done_bar));
    }
    __syncwarp();
    const bool ok = mbar_wait(smem_u32(&done_bar), 0, &abort_flag);
    tc_fence_after_sync();
    if (ok) {
        const int row = warp * 32 + lane;
        for (uint32_t c = 0; c < (L.n + 31) / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + c * 32, r);
            tmem_ld_wait();
            for (uint32_t q = 0; q < 32 && c * 32 + q < L.n; ++q) D[(size_t)row * L.n + c * 32 + q] = __uint_as_float(r[q]);
        }
    } else {
        if (lane == 0) atomicExch(status, 1);
        __nanosleep(100000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

// A operand from tensor memory: 128 threads (thread = row) write A[128][64] (bf16 pairs, as 32 words
// per row) into tensor-memory columns [256, 288) with tcgen05.st, one thread issues the four K = 16
// steps against a K-major shared-memory B tile [256][64], and D[128, 256] is read back.  `a_words` is
// [128][32] uint32: word w of a row = elements 2w (low half) and 2w + 1 (high half).
__global__ void __launch_bounds__(128, 1)
umma_tmem_a_kernel(const uint32_t* __restrict__ a_words, const uint8_t* __restrict__ b_img, float* __restrict__ D,
                   int* __restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t e = threadIdx.x * 16; e < kBBytes; e += blockDim.x * 16)
        *reinterpret_cast<uint4*>(smem + e) = *reinterpret_cast<const uint4*>(b_img + e);
    fence_proxy_async_smem();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    const int row = warp * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    for (int c = 0; c < 4; ++c) {
        uint32_t r[8];
        for (int q = 0; q < 8; ++q) r[q] = a_words[row * 32 + c * 8 + q];
        tmem_st_32x8(lane_addr + 256 + c * 8, r);
    }
    tmem_st_wait();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (threadIdx.x == 0) {
        const uint64_t b_desc = make_sdesc_sw128(16, 1024);
        const uint32_t idesc = make_idesc_bf16(256, false, false);
        for (int ks = 0; ks < 4; ++ks)
            mma_f16_ts(tmem_base, tmem_base + 256 + ks * 8, sdesc_at(b_desc, sbase + ks * 32), idesc, ks > 0 ? 1u : 0u);
        mma_commit(smem_u32(&done_bar));
    }
    __syncwarp();
    const bool ok = mbar_wait(smem_u32(&done_bar), 0, &abort_flag);
    tc_fence_after_sync();
    if (ok) {
        for (int c = 0; c < 8; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(lane_addr + c * 32, r);
            tmem_ld_wait();
            for (int q = 0; q < 32; ++q) D[(size_t)row * 256 + c * 32 + q] = __uint_as_float(r[q]);
        }
    } else {
        if (lane == 0) atomicExch(status, 1);
        __nanosleep(100000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

// Issue and completion cost of small MMAs: one or two threads (of different warps) each issue `reps`
// K = 16 MMAs with N columns (operands: zero-filled 128-byte-swizzled K-major tiles, the same for
// every MMA; accumulators: separate tensor-memory columns per thread) and commit.  Reports clock
// cycles: [0] issue loop of thread 0, [1] until thread 0's MMAs completed, [2], [3] the same for
// thread 1.
__global__ void __launch_bounds__(128, 1)
umma_rate_kernel(int n, int reps, int threads, int same_acc, long long* __restrict__ out, int* __restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t done_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t e = threadIdx.x * 16; e < 65536; e += blockDim.x * 16)
        *reinterpret_cast<uint4*>(smem + e) = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar[0]), 1);
        mbar_init(smem_u32(&done_bar[1]), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    if (lane == 0 && warp < threads) {
        const uint64_t desc = make_sdesc_sw128(16, 1024);
        const uint32_t idesc = make_idesc_bf16(n, false, false);
        const uint64_t a = sdesc_at(desc, sbase + warp * 16384), b = sdesc_at(desc, sbase + 32768);
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r)
            mma_f16_ss(tmem_base + warp * 256 + (same_acc ? 0 : (r & 7) * 32 * (n > 32 ? 0 : 1)), a + (uint64_t)((r & 3) * 2),
                       b + (uint64_t)((r & 3) * 2), idesc, 1u);
        mma_commit(smem_u32(&done_bar[warp]));
        const long long t1 = clock64();
        const bool ok = mbar_wait(smem_u32(&done_bar[warp]), 0, &abort_flag);
        const long long t2 = clock64();
        out[2 * warp] = t1 - t0;
        out[2 * warp + 1] = t2 - t0;
        if (!ok) atomicExch(status, 1);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512);
    }
}

// Register-only FMA loop for measuring the FP32 / FP64 FMA-pipe peaks the gather kernels are
// compared with: every thread runs `iters` rounds of 16 independent dependent-chain FMAs.
template <typename T>
__global__ void __launch_bounds__(256) fma_loop_kernel(T* __restrict__ out, int iters, T a, T b) {
    T v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = T(threadIdx.x + j) * T(1e-3);
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = fma(v[j], a, b);
    }
    T s = T(0);
#pragma unroll
    for (int j = 0; j < 16; ++j) s += v[j];
    out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = s;
}

// The same for the FP64 tensor-core instruction (mma.sync, the only FP64 matrix instruction the
// part has): every warp runs `iters` rounds of 8 independent accumulator tiles.
template <int SHAPE>
__global__ void __launch_bounds__(256) dmma_loop_kernel(double* __restrict__ out, int iters) {
    double c[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) c[j][q] = 0.0;
    double a[4], b[2];
#pragma unroll
    for (int q = 0; q < 4; ++q) a[q] = 1e-3 * (threadIdx.x + q);
    b[0] = 0.5, b[1] = 0.25;
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (SHAPE == 0) dmma::m8n8k4(c[j][0], c[j][1], a[0], b[0]);
            else dmma::m16n8k8(c[j], a, b);
        }
    }
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) s += c[j][q];
    out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = s;
}

// One warp, one instruction: the caller provides every lane's operand registers and reads every
// lane's accumulator registers, so a test can state the fragment layout it relies on in numpy.
__global__ void dmma_fragment_kernel(int shape, const double* __restrict__ a, const double* __restrict__ b,
                                     double* __restrict__ c) {
    const int lane = threadIdx.x;
    double cr[4] = {0.0, 0.0, 0.0, 0.0};
    if (shape == 0) {
        dmma::m8n8k4(cr[0], cr[1], a[lane], b[lane]);
    } else {
        double ar[4], br[2];
        for (int q = 0; q < 4; ++q) ar[q] = a[lane * 4 + q];
        for (int q = 0; q < 2; ++q) br[q] = b[lane * 2 + q];
        dmma::m16n8k8(cr, ar, br);
    }
    for (int q = 0; q < 4; ++q) c[lane * 4 + q] = cr[q];
}
}  // namespace
}  // namespace kanb200

// FP64 matrix-instruction loop: shape 0 = m8n8k4 (256 FMAs per warp instruction), 1 = m16n8k8
// (1024).  Executed FMAs: blocks * 8 warps * iters * 8 * that.  `out` holds blocks * 256 doubles.
extern "C" __attribute__((visibility("default")))
int kanb200_selftest_dmma_loop(int shape, int blocks, int iters, void* out, void* stream) {
    using namespace kanb200;
    if (blocks < 1 || blocks > 65535 || iters < 1 || !out || shape < 0 || shape > 1) return -1;
    if (shape == 0) dmma_loop_kernel<0><<<blocks, 256, 0, (cudaStream_t)stream>>>((double*)out, iters);
    else dmma_loop_kernel<1><<<blocks, 256, 0, (cudaStream_t)stream>>>((double*)out, iters);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One warp-wide FP64 matrix instruction on caller-provided fragments: a holds 32 x (1 | 4) doubles,
// b 32 x (1 | 2), c receives 32 x 4 (shape 0 fills the first two of each lane).
extern "C" __attribute__((visibility("default")))
int kanb200_selftest_dmma_fragments(int shape, const double* a, const double* b, double* c, void* stream) {
    using namespace kanb200;
    if (shape < 0 || shape > 1 || !a || !b || !c) return -1;
    dmma_fragment_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(shape, a, b, c);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Launches blocks x 256 threads of the FMA loop (dtype 0 = float, 1 = double); the caller times it
// with events.  FMAs executed: blocks * 256 * iters * 16.  `out` holds blocks * 256 elements.
extern "C" __attribute__((visibility("default")))
int kanb200_selftest_fma_loop(int dtype, int blocks, int iters, void* out, void* stream) {
    using namespace kanb200;
    if (blocks < 1 || blocks > 65535 || iters < 1 || !out) return -1;
    if (dtype == 0)
        fma_loop_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float*)out, iters, 0.999f, 1e-3f);
    else
        fma_loop_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((double*)out, iters, 0.999, 1e-3);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" __attribute__((visibility("default")))
int kanb200_selftest_umma_layout(int layout, const void* a_img, const void* b_img, float* D, int* status,
                                 void* stream) {
    using namespace kanb200;
    if ((layout != kLayoutKMajor && layout != kLayoutMnMajor) || !a_img || !b_img || !D || !status) return -1;
    const int smem = (int)(kABytes + kBBytes);
    cudaError_t e = cudaFuncSetAttribute(umma_layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return -4;
    umma_layout_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(reinterpret_cast<const uint8_t*>(a_img),
                                                                reinterpret_cast<const uint8_t*>(b_img), layout, D,
                                                                status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// D[128, n] of `ksteps` K = 16 steps with caller-named layout parameters (16 integers in the order
// of GeneralLayout); operands at most 32 KB each, n a multiple of 16 up to 256.
extern "C" __attribute__((visibility("default")))
int kanb200_selftest_umma_general(const void* a_img, const void* b_img, const unsigned* params, float* D,
                                  int* status, void* stream) {
    using namespace kanb200;
    if (!a_img || !b_img || !params || !D || !status) return -1;
    GeneralLayout L;
    L.a_bytes = params[0]; L.b_bytes = params[1]; L.a_mn = params[2]; L.b_mn = params[3];
    L.a_lbo = params[4]; L.a_sbo = params[5]; L.a_step = params[6]; L.a_off = params[7];
    L.b_lbo = params[8]; L.b_sbo = params[9]; L.b_step = params[10]; L.b_off = params[11];
    L.n = params[12]; L.ksteps = params[13];
    if (L.a_bytes > 32768 || L.b_bytes > 32768 || (L.a_bytes & 15) || (L.b_bytes & 15) || L.n < 16 || L.n > 256 ||
        (L.n & 15) || L.ksteps < 1 || L.ksteps > 16)
        return -1;
    const uint64_t a_last = (uint64_t)L.a_off + (uint64_t)(L.ksteps - 1) * L.a_step;
    const uint64_t b_last = (uint64_t)L.b_off + (uint64_t)(L.ksteps - 1) * L.b_step;
    if (a_last >= 32768 || b_last >= 32768) return -1;
    const int smem = 65536;
    cudaError_t e = cudaFuncSetAttribute(umma_general_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return -4;
    umma_general_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(reinterpret_cast<const uint8_t*>(a_img),
                                                                 reinterpret_cast<const uint8_t*>(b_img), L, D, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// See umma_rate_kernel: n columns (16 .. 256), reps MMAs per thread, 1 or 2 issuing threads,
// same_acc = every MMA of a thread accumulates into the same columns.  out receives 4 cycle counts.
extern "C" __attribute__((visibility("default")))
int kanb200_selftest_umma_rate(int n, int reps, int threads, int same_acc, long long* out, int* status, void* stream) {
    using namespace kanb200;
    if (n < 16 || n > 256 || (n & 15) || reps < 1 || reps > 4096 || threads < 1 || threads > 2 || !out || !status) return -1;
    const int smem = 65536;
    cudaError_t e = cudaFuncSetAttribute(umma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return -4;
    umma_rate_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(n, reps, threads, same_acc, out, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// See umma_tmem_a_kernel: a_words [128][32] uint32 (bf16 pairs), b_img the K-major image of B [256][64].
extern "C" __attribute__((visibility("default")))
int kanb200_selftest_umma_tmem_a(const void* a_words, const void* b_img, float* D, int* status, void* stream) {
    using namespace kanb200;
    if (!a_words || !b_img || !D || !status) return -1;
    const int smem = (int)kBBytes;
    cudaError_t e = cudaFuncSetAttribute(umma_tmem_a_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return -4;
    umma_tmem_a_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(reinterpret_cast<const uint32_t*>(a_words),
                                                                reinterpret_cast<const uint8_t*>(b_img), D, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
