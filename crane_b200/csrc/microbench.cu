// Two measurements of the machine that the kernels' designs lean on (a library of its own, built
// only when `python -m crane_b200.profiling hardware` asks for it):
//   * how many cycles one thread needs per tcgen05.mma of 128 x N x 16 (bf16) issued back to back on
//     operands that lie in shared memory;
//   * what a barrier across the SMs costs (one CTA per SM, cooperative launch: a release-add on a
//     counter in global memory, then acquire-loads until all have arrived).
// Every wait is bounded; a wait that runs out is reported, nothing spins for ever.
#include <cstdint>
#include <cuda_runtime.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// K-major operand, rows of 128 bytes, 128-byte swizzle (as in gemm_tcgen05.cu)
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// out[0]: cycles of the issuing loop, out[1]: cycles until the last product is complete, out[2]: 1 if it completed
template <int N>
__global__ void __launch_bounds__(128) mma_issue_kernel(long long* out, int reps) {
    extern __shared__ __align__(1024) uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < (16384 + N * 128) / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x3c003c00u;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = slot;
    if (threadIdx.x == 0) {
        const uint64_t da = desc_sw128(smem_u32(smem)), db = desc_sw128(smem_u32(smem + 16384));
        const uint32_t id = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t acc = (r > 0 || kk > 0) ? 1u : 0u;
                asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                             ::"r"(tmem), "l"(da + 2 * kk), "l"(db + 2 * kk), "r"(id), "r"(acc) : "memory");
            }
        }
        const long long t1 = clock64();
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
        bool done = false;
        for (int i = 0; i < (1 << 24) && !done; ++i) done = try_wait(smem_u32(&bar), 0);
        const long long t2 = clock64();
        out[0] = t1 - t0; out[1] = t2 - t0; out[2] = done ? 1 : 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
}

__global__ void __launch_bounds__(128) grid_barrier_kernel(unsigned* counter, long long* out, int rounds, int* err) {
    const unsigned n = gridDim.x;
    __shared__ int bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    const long long t0 = clock64();
    for (int r = 0; r < rounds; ++r) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
            const unsigned target = (unsigned)(r + 1) * n;
            unsigned v = 0;
            int spins = 0;
            do {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            } while (v < target && ++spins < (1 << 22));
            if (v < target) { bad = 1; atomicOr(err, 1); }
        }
        __syncthreads();
        if (bad) break;
    }
    if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = clock64() - t0;
}

template <int N>
int run_mma_issue(long long* out, int reps, cudaStream_t st) {
    const size_t smem = 16384 + N * 128 + 1024;
    if (cudaFuncSetAttribute(mma_issue_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return (int)cudaGetLastError();
    mma_issue_kernel<N><<<1, 128, smem, st>>>(out, reps);
    return crane_launch_status();
}

}  // namespace

// out: 3 long longs on the device (see the kernel).  n: 64, 128 or 256.  4 * reps products are issued.
CRANE_API int crane_microbench_mma_issue(int n, int reps, long long* out, cudaStream_t st) {
    switch (n) {
        case 64: return run_mma_issue<64>(out, reps, st);
        case 128: return run_mma_issue<128>(out, reps, st);
        case 256: return run_mma_issue<256>(out, reps, st);
    }
    return (int)cudaErrorInvalidValue;
}

// counter (zeroed), out (1 long long: cycles of all rounds), err (zeroed; 1 if a wait ran out) on the device.
// ctas must not exceed the number of SMs (one CTA each; the launch is cooperative, so all are resident).
CRANE_API int crane_microbench_grid_barrier(int ctas, int rounds, unsigned* counter, long long* out, int* err,
                                            cudaStream_t st) {
    int dev = 0, sms = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop || ctas < 1 || ctas > sms || rounds < 1) return (int)cudaErrorInvalidValue;
    void* args[] = {&counter, &out, &rounds, &err};
    const cudaError_t rc = cudaLaunchCooperativeKernel((void*)grid_barrier_kernel, dim3(ctas), dim3(128), args, 0, st);
    const cudaError_t last = cudaGetLastError();
    return rc != cudaSuccess ? (int)rc : (int)last;
}
