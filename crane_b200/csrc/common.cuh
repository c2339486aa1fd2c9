// Shared device helpers for the sm_100a kernels of this engine.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define CRANE_API extern "C" __attribute__((visibility("default")))

// Bits of the device-side error word.  Kernels never trap: they record what
// went wrong, skip the access and return; the host reads the word after a step.
enum CraneErr : int {
    CRANE_ERR_TOKEN_RANGE = 1,      // token id outside the vocabulary
    CRANE_ERR_PAGE_RANGE = 2,       // block-table entry outside the page pool
    CRANE_ERR_POSITION_RANGE = 4,   // position outside the rotary table
    CRANE_ERR_WAIT_TIMEOUT = 8,     // a bounded mbarrier wait ran out
    CRANE_ERR_SLOT_RANGE = 16,
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole block of up to 1024 threads; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // scratch may still be read from an earlier call
    if (lane == 0) scratch32[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch32[lane] : 0.f;
    return warp_sum(t);
}

// How a mixer's heads are rotated and normalised.  The defaults are Hunyuan Dense's: the whole head
// rotated in the contiguous-halves pairing, RMSNorm after the rotation, plain weights.
struct RopeParams {
    int rotary_dim;      // the leading elements of a head that are rotated (even, <= head size)
    int interleaved;     // 0: element i pairs with i + rotary_dim / 2;  1: 2i with 2i + 1
    int norm_first;      // 0: per-head RMSNorm after the rotation;  1: before it
    float norm_offset;   // the norm multiplies by (norm_offset + w): 0 plain, 1 for weights stored as w - 1
};
static inline bool rope_is_default(const RopeParams& p, int d) {
    return p.rotary_dim == d && !p.interleaved && !p.norm_first && p.norm_offset == 0.f;
}
// A head of d elements seen as d / 2 slots of two elements: slot i < rotary_dim / 2 holds a rotated
// pair (its angle is column i of the tables), the other slots hold the neighbours behind the rotated part.
__device__ __forceinline__ void rope_slot(const RopeParams& p, int i, int& ea, int& eb, bool& rot) {
    const int hr = p.rotary_dim >> 1;
    rot = i < hr;
    if (rot) {
        ea = p.interleaved ? 2 * i : i;
        eb = p.interleaved ? 2 * i + 1 : i + hr;
    } else {
        ea = p.rotary_dim + 2 * (i - hr);
        eb = ea + 1;
    }
}
// One head row by one warp for any RopeParams: `load(e)` gives element e as float, `store(e, v)`
// takes the result.  cos/sin tables are [positions][rotary_dim / 2].  nw: the norm's weight or null.
template <int MAXS, typename Load, typename Store>
__device__ __forceinline__ void rope_norm_general(const RopeParams& rp, int d, int pos, bool rotate,
                                                  const float* __restrict__ cos_tab,
                                                  const float* __restrict__ sin_tab,
                                                  const float* __restrict__ nw, float eps, int lane,
                                                  Load load, Store store) {
    const int hr = rp.rotary_dim >> 1, slots = d >> 1;
    float a[MAXS], b[MAXS];
    float ss = 0.f;
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
        const int i = lane + 32 * s;
        a[s] = b[s] = 0.f;
        if (i < slots) {
            int ea, eb; bool rot;
            rope_slot(rp, i, ea, eb, rot);
            a[s] = load(ea);
            b[s] = load(eb);
            ss += a[s] * a[s] + b[s] * b[s];
        }
    }
    if (nw != nullptr && rp.norm_first) {
        unsigned m = 0xffffffffu;
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(m, ss, o);
        const float rstd = rsqrtf(ss / (float)d + eps);
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
            const int i = lane + 32 * s;
            if (i < slots) {
                int ea, eb; bool rot;
                rope_slot(rp, i, ea, eb, rot);
                a[s] = a[s] * rstd * (rp.norm_offset + nw[ea]);
                b[s] = b[s] * rstd * (rp.norm_offset + nw[eb]);
            }
        }
    }
    ss = 0.f;
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
        const int i = lane + 32 * s;
        if (i < slots) {
            if (rotate && i < hr) {
                const float c = cos_tab[(long long)pos * hr + i], sn = sin_tab[(long long)pos * hr + i];
                const float x1 = a[s], x2 = b[s];
                a[s] = x1 * c - x2 * sn;
                b[s] = x2 * c + x1 * sn;
            }
            ss += a[s] * a[s] + b[s] * b[s];
        }
    }
    float rstd = 1.f;
    const bool after = nw != nullptr && !rp.norm_first;
    if (after) {
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        rstd = rsqrtf(ss / (float)d + eps);
    }
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
        const int i = lane + 32 * s;
        if (i < slots) {
            int ea, eb; bool rot;
            rope_slot(rp, i, ea, eb, rot);
            store(ea, after ? a[s] * rstd * (rp.norm_offset + nw[ea]) : a[s]);
            store(eb, after ? b[s] * rstd * (rp.norm_offset + nw[eb]) : b[s]);
        }
    }
}

// Programmatic dependent launch: a kernel launched with the attribute may start
// while the kernel before it in the stream is still running.  It must not touch
// anything that kernel (or one before it) writes or reads-then-overwrites until
// it has called pdl_wait(), which returns once all earlier kernels are complete
// and their writes visible.  pdl_launch_dependents() lets the NEXT kernel start
// early in the same way.  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

static inline int crane_launch_status() { return (int)cudaGetLastError(); }

// 1: kernels of a decoder step are launched with programmatic dependent launch.
extern int g_crane_pdl;

template <typename... KArgs, typename... Args>
static inline int crane_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_crane_pdl ? 1 : 0;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
    const cudaError_t last = cudaGetLastError();        // read, and with that cleared, in either case:
    return rc != cudaSuccess ? (int)rc : (int)last;     // a refused launch must not fail the next one too
}

// The same for a kernel whose CTAs form thread-block clusters of `cluster` CTAs.
template <typename... KArgs, typename... Args>
static inline int crane_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       dim3 cluster, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_crane_pdl ? 2 : 1;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
    const cudaError_t last = cudaGetLastError();        // read, and with that cleared, in either case:
    return rc != cudaSuccess ? (int)rc : (int)last;     // a refused launch must not fail the next one too
}
