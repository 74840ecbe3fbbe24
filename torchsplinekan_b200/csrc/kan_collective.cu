// Gradient all-reduce over NVLink / NVSwitch for batch-sharded training.
//
// Every rank owns one allocation of the same size ("symmetric" memory) that all ranks of the
// node have mapped: [payload floats | signal pad].  One launch per rank sums the payload over
// the ranks and leaves the result in every rank's copy:
//
//   1. barrier   every rank's payload is complete (its producers ran earlier on the stream)
//   2. reduce    rank r owns the r-th slice of the payload.  With a multicast mapping
//                (NVSwitch) one multimem.ld_reduce returns the sum over all ranks, computed in
//                the switch, and one multimem.st writes it to all ranks.  Without it the owner
//                loads the slice from every peer in rank order, adds, and stores to every peer.
//   3. barrier   all slices have landed everywhere
//
// Block b of rank r only talks to block b of the other ranks: signal word [b][src] of a rank's
// pad is raised by block b of rank src (CAS 0 -> 1) and lowered by the owner (CAS 1 -> 0), so
// the pad needs no reset between calls.  Every spin has a time limit (ten seconds unless set otherwise); when it runs out
// the kernel records kStatusTimeout in the caller's status word and returns (the pad is then
// in an undefined state and must be zeroed before the next call).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kan_b200.h"
#include "kan_internal.h"

namespace kanb200 {
namespace {

constexpr int AR_THREADS = 512;
constexpr int AR_UNROLL = 8;
constexpr int kArTimeout = 1;
// Limit of one wait on another rank.  Ranks of a job drift apart by much more than a kernel's
// run time (first-call set-up, host scheduling), so the default is generous; it is still a bound.
static unsigned long long g_wait_limit_ns = 10000000000ull;

struct PeerTable {
    void* base[KANB200_MAX_RANKS];
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t cas_release_sys(uint32_t* addr, uint32_t expect, uint32_t value) {
    uint32_t old;
    asm volatile("atom.global.release.sys.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old) : "l"(addr), "r"(expect), "r"(value) : "memory");
    return old;
}
__device__ __forceinline__ uint32_t cas_acquire_sys(uint32_t* addr, uint32_t expect, uint32_t value) {
    uint32_t old;
    asm volatile("atom.global.acquire.sys.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old) : "l"(addr), "r"(expect), "r"(value) : "memory");
    return old;
}

// Block-level barrier with the same block of every other rank.  Returns false after a timeout.
__device__ bool rank_barrier(const PeerTable& peers, size_t pad_off, int rank, int world, int block,
                             unsigned long long limit_ns, int* status, int* abort_flag) {
    __threadfence_system();                    // this thread's stores, visible to the peers
    __syncthreads();
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
        const int p = threadIdx.x;
        uint32_t* remote = reinterpret_cast<uint32_t*>(static_cast<char*>(peers.base[p]) + pad_off) +
                           (size_t)block * world + rank;
        uint32_t* local = reinterpret_cast<uint32_t*>(static_cast<char*>(peers.base[rank]) + pad_off) +
                          (size_t)block * world + p;
        const unsigned long long t0 = global_timer_ns();
        bool ok = false;
        do {
            if (cas_release_sys(remote, 0u, 1u) == 0u) { ok = true; break; }
            __nanosleep(64);
        } while (global_timer_ns() - t0 < limit_ns);
        if (ok) {
            ok = false;
            do {
                if (cas_acquire_sys(local, 1u, 0u) == 1u) { ok = true; break; }
                __nanosleep(64);
            } while (global_timer_ns() - t0 < limit_ns);
        }
        if (!ok) {
            atomicExch(status, kArTimeout);
            atomicExch(abort_flag, 1);
        }
    }
    __syncthreads();
    return *reinterpret_cast<volatile int*>(abort_flag) == 0;
}

__device__ __forceinline__ float4 multimem_ld_reduce_add(const float4* mc) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st(float4* mc, const float4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer(float4* p, const float4& v) {
    asm volatile("st.volatile.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Up to 4 ranges of one allocation reduced by one launch (the gradients of a range of output rows
// of a layer are three ranges of its bucket: spline weight, scaler, base weight).
struct Segments {
    size_t off[KANB200_MAX_SEGMENTS];      // byte offset of the range within the allocation
    size_t n4[KANB200_MAX_SEGMENTS];       // 16-byte pieces
    int count;
};

// gridDim.x blocks per rank; gridDim.y > 1 runs several ranks of one device in a single launch
// (all blocks co-resident), which is how the protocol is exercised on one GPU.
template <bool MULTIMEM>
__global__ void __launch_bounds__(AR_THREADS)
allreduce_sum_kernel(PeerTable peers, char* mc_base, Segments segs, size_t pad_off,
                     int rank0, int world, float scale, unsigned long long limit_ns, int* status) {
    __shared__ int abort_flag;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    const int rank = rank0 + blockIdx.y;
    const int block = blockIdx.x;
    if (!rank_barrier(peers, pad_off, rank, world, block, limit_ns, status, &abort_flag)) return;

    for (int sg = 0; sg < segs.count; ++sg) {
        const size_t n4 = segs.n4[sg], payload_off = segs.off[sg];
        float4* mc_payload = reinterpret_cast<float4*>(mc_base + payload_off);
        const size_t per = (n4 + world - 1) / world;
        const size_t lo = (size_t)rank * per;
        size_t hi = lo + per;
        if (hi > n4) hi = n4;
        // AR_UNROLL independent 16-byte pieces per thread are in flight at a time: a load through
        // the switch takes microseconds, so bandwidth comes from the number of outstanding requests.
        const size_t step = (size_t)gridDim.x * blockDim.x;
        for (size_t i0 = lo + (size_t)block * blockDim.x + threadIdx.x; i0 < hi; i0 += step * AR_UNROLL) {
            float4 v[AR_UNROLL];
#pragma unroll
            for (int u = 0; u < AR_UNROLL; ++u) {
                const size_t i = i0 + (size_t)u * step;
                if (i < hi) {
                    if (MULTIMEM) {
                        v[u] = multimem_ld_reduce_add(mc_payload + i);
                    } else {
                        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int p = 0; p < world; ++p) {
                            const float4 a = ld_peer(
                                reinterpret_cast<const float4*>(static_cast<char*>(peers.base[p]) + payload_off) + i);
                            v[u].x += a.x; v[u].y += a.y; v[u].z += a.z; v[u].w += a.w;
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < AR_UNROLL; ++u) {
                const size_t i = i0 + (size_t)u * step;
                if (i < hi) {
                    float4 r = v[u];
                    r.x *= scale; r.y *= scale; r.z *= scale; r.w *= scale;
                    if (MULTIMEM) {
                        multimem_st(mc_payload + i, r);
                    } else {
                        for (int p = 0; p < world; ++p)
                            st_peer(reinterpret_cast<float4*>(static_cast<char*>(peers.base[p]) + payload_off) + i, r);
                    }
                }
            }
        }
    }
    rank_barrier(peers, pad_off, rank, world, block, limit_ns, status, &abort_flag);
}

}  // namespace

void allreduce_set_wait_limit_ms(unsigned ms) { g_wait_limit_ns = (unsigned long long)ms * 1000000ull; }

size_t allreduce_pad_bytes(int world, int blocks) {
    return ((size_t)world * blocks * sizeof(uint32_t) + 255) / 256 * 256;
}

cudaError_t allreduce_sum(void* const* peer_bases, void* multicast_base, const size_t* offsets, const size_t* n_floats,
                          int n_segments, size_t pad_off, int rank, int world, int local_ranks, int blocks,
                          int threads, float scale, int* status, cudaStream_t st) {
    PeerTable t;
    for (int p = 0; p < KANB200_MAX_RANKS; ++p) t.base[p] = p < world ? peer_bases[p] : nullptr;
    Segments segs;
    segs.count = n_segments;
    for (int i = 0; i < KANB200_MAX_SEGMENTS; ++i) {
        segs.off[i] = i < n_segments ? offsets[i] : 0;
        segs.n4[i] = i < n_segments ? n_floats[i] / 4 : 0;
    }
    dim3 grid((unsigned)blocks, (unsigned)local_ranks);
    if (multicast_base)
        allreduce_sum_kernel<true><<<grid, threads, 0, st>>>(t, static_cast<char*>(multicast_base), segs, pad_off,
                                                            rank, world, scale, g_wait_limit_ns, status);
    else
        allreduce_sum_kernel<false><<<grid, threads, 0, st>>>(t, nullptr, segs, pad_off, rank, world, scale,
                                                             g_wait_limit_ns, status);
    return cudaGetLastError();
}

}  // namespace kanb200
