// Self-test kernel for the shared-memory operand layouts of tcgen05.mma.
//
// One CTA copies two caller-built byte images into shared memory, issues
// `ksteps` MMAs (M = 128, N = ncols, K = 16 each) with caller-given matrix and
// instruction descriptors and writes the fp32 accumulator out.  The test-suite
// builds the images for the K-major and MN-major 128-byte-swizzle layouts used
// by the production kernels and checks the product against numpy, so a wrong
// descriptor shows up as a failed small test instead of a wrong large result.
#include "kan_internal.h"
#include "kan_tc_ptx.cuh"

namespace kanb200 {

namespace {
using namespace ptx;

__global__ void __launch_bounds__(128, 1)
umma_probe_kernel(const uint8_t* __restrict__ a_img, uint32_t a_bytes, const uint8_t* __restrict__ b_img,
                  uint32_t b_bytes, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, int ksteps,
                  uint32_t a_step, uint32_t b_step, int ncols, float* __restrict__ D, int* __restrict__ status) {
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
}  // namespace

cudaError_t umma_probe(const void* a_img, uint32_t a_bytes, const void* b_img, uint32_t b_bytes,
                       uint64_t a_desc, uint64_t b_desc, uint32_t idesc, int ksteps, uint32_t a_step,
                       uint32_t b_step, int ncols, float* D, int* status, cudaStream_t st) {
    const size_t smem = ((a_bytes + 1023u) & ~1023u) + ((b_bytes + 1023u) & ~1023u);
    if (smem > 200 * 1024 || ncols % 32 != 0 || ncols < 32 || ncols > 256) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    umma_probe_kernel<<<1, 128, smem, st>>>(reinterpret_cast<const uint8_t*>(a_img), a_bytes,
                                            reinterpret_cast<const uint8_t*>(b_img), b_bytes, a_desc, b_desc,
                                            idesc, ksteps, a_step, b_step, ncols, D, status);
    return cudaGetLastError();
}

}  // namespace kanb200
