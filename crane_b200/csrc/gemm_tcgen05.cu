// bf16 matrix product on the 5th-generation tensor cores of sm_100a:
//   D[a, b] = sum_k A[a, k] * B[b, k]        A [rows_a, K], B [rows_b, K], both K-contiguous
// Operands travel global -> shared memory by TMA (128-byte swizzle), the
// product is issued by one thread as tcgen05.mma with the float accumulator in
// tensor memory, and four warps read the accumulator back with tcgen05.ld for
// the epilogue.  One CTA computes one 128 x BN tile over one slice of K.
//
// Two ways to use it for y = x W^T (crane-core/src/models/hunyuan_dense/
// modeling.rs:273-330: weights are [out, in]):
//   * many tokens:  A = x, B = W, BN = 128 or 256, output row-major [token, feature];
//   * few tokens:   A = W, B = x ("swap-AB": the 128-wide side of the MMA is
//     filled by weight rows, the narrow side holds 16..64 tokens), output
//     written transposed so that it is again [token, feature].
// With split_k > 1 every slice writes its float partial sums [slice][row][col]
// and the consumer adds them (see GemmOut in elementwise.cu).
//
// Launched with programmatic dependent launch: the first tiles of the weights
// are requested before the kernel waits for its predecessor (see the producer).
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records
// CRANE_ERR_WAIT_TIMEOUT, all roles leave their loops, tensor memory is freed
// and the kernel returns.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;          // rows of A per tile = MMA M
constexpr int BK = 64;           // bf16 elements per k-block = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192; // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..5: epilogue
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA's abort flag) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart (stride byte offset), leading byte
// offset 1 (unused for swizzled K-major), descriptor version 1, layout 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

struct GemmParams {
    int rows_a, rows_b, k;          // extents
    void* out;                      // bf16 or float, see template flags
    long long ld_out;               // elements between consecutive rows of the output
    long long split_stride;         // elements between consecutive slices (split_k > 1)
    const float* bias;              // over the feature dimension, or null
    int* err;
    const uint8_t* prefetch;        // what the NEXT product of the step will stream (its weights), or null:
    long long prefetch_bytes;       // asked into L2 by this kernel's idle warp as soon as it starts
};

// The kernels of a decode step run one after the other, each for a few microseconds, and each begins
// by waiting for its operands to arrive from DRAM.  A product that is told what the next product
// will stream asks for it at once (a hint: bulk prefetches into L2, no data comes to the SM, nothing
// waits for them), so that DRAM keeps streaming through the short kernels between the two and the
// next product finds its weights in L2.
__device__ __forceinline__ void prefetch_l2(const GemmParams& p, int lane) {
    if (p.prefetch == nullptr) return;
    constexpr long long PIECE = 16384;
    const long long ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
    const long long cta = blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z);
    const long long pieces = (p.prefetch_bytes + PIECE - 1) / PIECE;
    const long long per = (pieces + ctas - 1) / ctas;
    const long long end = min(pieces, (cta + 1) * per);
    for (long long i = cta * per + lane; i < end; i += 32) {
        const long long off = i * PIECE;
        const uint32_t bytes = (uint32_t)min(PIECE, p.prefetch_bytes - off) & ~15u;
        if (bytes)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.prefetch + off), "r"(bytes) : "memory");
    }
}

// OUT_F32: float output (else bf16).  TRANSPOSED: element (a, b) goes to out[b * ld + a].
template <int BN, int STAGES, bool OUT_F32, bool TRANSPOSED>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment is what the 128-byte swizzle pattern is anchored to
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint64_t* bars = (uint64_t*)(smem + STAGES * (A_BYTES + B_BYTES));
    uint64_t* full = bars;                    // [STAGES] operands of a stage have landed
    uint64_t* empty = bars + STAGES;          // [STAGES] the MMAs that read a stage are done
    uint64_t* acc_ready = bars + 2 * STAGES;  // the whole accumulator is done
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * BM, b0 = blockIdx.y * BN;
    // the k-blocks are dealt out to the slices as evenly as they go
    const int num_kb_total = (p.k + BK - 1) / BK;
    const int kb_begin = (int)(((long long)blockIdx.z * num_kb_total) / gridDim.z);
    const int kb_end = (int)(((long long)(blockIdx.z + 1) * num_kb_total) / gridDim.z);
    const int num_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(acc_ready), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        // The weights (A when transposed, else B) depend on no earlier kernel: their
        // first tiles are requested before waiting for the kernel that produces the
        // activations, so the stream of weights starts while that kernel still runs.
        const int pre = min(num_kb, STAGES);
        for (int i = 0; i < pre; ++i) {
            const uint32_t bar = smem_u32(&full[i]);
            mbar_expect_tx(bar, A_BYTES + B_BYTES);
            const int k0 = (kb_begin + i) * BK;
            if (TRANSPOSED) tma_load_2d(smem_u32(smem_a + i * A_BYTES), &map_a, bar, k0, a0);
            else tma_load_2d(smem_u32(smem_b + i * B_BYTES), &map_b, bar, k0, b0);
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
            const uint32_t bar = smem_u32(&full[i]);
            const int k0 = (kb_begin + i) * BK;
            if (TRANSPOSED) tma_load_2d(smem_u32(smem_b + i * B_BYTES), &map_b, bar, k0, b0);
            else tma_load_2d(smem_u32(smem_a + i * A_BYTES), &map_a, bar, k0, a0);
        }
        for (int i = pre; i < num_kb; ++i) {
            const int s = i % STAGES;
            const uint32_t parity = ((i / STAGES) & 1) ^ 1;
            if (!mbar_wait(smem_u32(&empty[s]), parity, abort_flag)) break;
            const uint32_t bar = smem_u32(&full[s]);
            mbar_expect_tx(bar, A_BYTES + B_BYTES);
            const int k0 = (kb_begin + i) * BK;
            tma_load_2d(smem_u32(smem_a + s * A_BYTES), &map_a, bar, k0, a0);
            tma_load_2d(smem_u32(smem_b + s * B_BYTES), &map_b, bar, k0, b0);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = instr_desc_bf16(BN);
        for (int i = 0; i < num_kb; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(smem_u32(&full[s]), (i / STAGES) & 1, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc_sw128(smem_u32(smem_a + s * A_BYTES));
            const uint64_t db = smem_desc_sw128(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                // 16 elements further along K: 32 bytes, 2 in descriptor units of 16 bytes
                umma_bf16(tmem_base, da + 2 * kk, db + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&empty[s]));
        }
        umma_commit(smem_u32(acc_ready));
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        if (warp == 2) prefetch_l2(p, lane);               // idle until the accumulator is done
        // a warp may touch the 32 lanes of tensor memory given by its index modulo 4
        const int quarter = warp & 3;
        const bool ok = num_kb == 0 || mbar_wait(smem_u32(acc_ready), 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int a = a0 + quarter * 32 + lane;            // this thread's row of A
        const bool split = gridDim.z > 1;
        const bool with_bias = p.bias != nullptr && blockIdx.z == 0;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                if (num_kb > 0) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
                if (a >= p.rows_a) continue;
                if (!TRANSPOSED && !split && b0 + c0 + 16 <= p.rows_b) {
                    // 16 consecutive features of one token: whole 16-byte stores when aligned
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        v[j] = __uint_as_float(r[j]);
                        if (with_bias) v[j] += p.bias[b0 + c0 + j];
                    }
                    const long long idx = (long long)a * p.ld_out + b0 + c0;
                    if (OUT_F32) {
                        float* dst = (float*)p.out + idx;
                        if (((uintptr_t)dst & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *(float4*)(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) dst[j] = v[j];
                        }
                    } else {
                        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + idx;
                        if (((uintptr_t)dst & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 16; j += 8) {
                                uint4 w;
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                w.x = *(uint32_t*)&h0; w.y = *(uint32_t*)&h1;
                                w.z = *(uint32_t*)&h2; w.w = *(uint32_t*)&h3;
                                *(uint4*)(dst + j) = w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) dst[j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                    continue;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int b = b0 + c0 + j;
                    if (b >= p.rows_b) break;
                    float v = __uint_as_float(r[j]);
                    const int feature = TRANSPOSED ? a : b;
                    if (with_bias) v += p.bias[feature];
                    const long long idx = TRANSPOSED ? (long long)b * p.ld_out + a
                                                     : (long long)a * p.ld_out + b;
                    if (split)
                        ((float*)p.out)[(long long)blockIdx.z * p.split_stride + idx] = v;
                    else if (OUT_F32)
                        ((float*)p.out)[idx] = v;
                    else
                        ((__nv_bfloat16*)p.out)[idx] = __float2bfloat16_rn(v);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicOr(p.err, CRANE_ERR_WAIT_TIMEOUT);
        // copies that were issued may still be landing: give them time before the CTA ends
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Many tokens: a persistent kernel.  One CTA per SM walks over output tiles
// (A rows fastest, so CTAs that run together share a tile of weights in L2).
// The accumulator is double-buffered in tensor memory: while the four epilogue
// warps drain tile i, the MMA warp already fills the other buffer with tile
// i + 1, and the TMA warp runs ahead of both across tile borders.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// 32 consecutive accumulator columns of row `a` (values r[], first column b_first) go out:
// with bias, as float or bf16, in whole 16-byte stores where the row allows it, or as
// silu(gate) * up of 16 features.
template <bool OUT_F32, bool SILU>
__device__ __forceinline__ void store_chunk32(const GemmParams& p, const uint32_t (&r)[32], int a, int b_first) {
    if (SILU) {
        // columns 0..15 of the chunk: gate, 16..31: up, of features b_first / 2 + 0..15
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (long long)a * p.ld_out + (b_first >> 1);
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float g = __uint_as_float(r[j]), u = __uint_as_float(r[16 + j]);
            // the result is rounded to bf16: the approximate exp and division (each good to a
            // few units in the last place of a float) are far inside that, and a third as long
            v[j] = __fdividef(g, 1.f + __expf(-g)) * u;
        }
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
            uint4 w;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
            w.x = *(uint32_t*)&h0; w.y = *(uint32_t*)&h1;
            w.z = *(uint32_t*)&h2; w.w = *(uint32_t*)&h3;
            *(uint4*)(dst + j) = w;
        }
        return;
    }
    const long long idx = (long long)a * p.ld_out + b_first;
    const bool whole = b_first + 32 <= p.rows_b;
    if (OUT_F32) {
        float* dst = (float*)p.out + idx;
        if (whole && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                       __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                if (p.bias) { v.x += p.bias[b_first + j]; v.y += p.bias[b_first + j + 1];
                              v.z += p.bias[b_first + j + 2]; v.w += p.bias[b_first + j + 3]; }
                *(float4*)(dst + j) = v;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (b_first + j < p.rows_b)
                    dst[j] = __uint_as_float(r[j]) + (p.bias ? p.bias[b_first + j] : 0.f);
        }
    } else {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + idx;
        if (whole && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                float v[8];
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    v[q] = __uint_as_float(r[j + q]) + (p.bias ? p.bias[b_first + j + q] : 0.f);
                uint4 w;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
                w.x = *(uint32_t*)&h0; w.y = *(uint32_t*)&h1;
                w.z = *(uint32_t*)&h2; w.w = *(uint32_t*)&h3;
                *(uint4*)(dst + j) = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (b_first + j < p.rows_b)
                    dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]) +
                                                 (p.bias ? p.bias[b_first + j] : 0.f));
        }
    }
}

// SILU: the B rows (weights) come in blocks of 32 = 16 gate rows then the 16 up
// rows of the same features; the epilogue writes silu(gate) * up, half as many
// columns as the product has (silu(x) = x / (1 + exp(-x)) in float:
// crane-core/kernels/fused_ops.cu:39-42, 112-130).
//
// MT: how many 128-row blocks of A a tile has.  With MT = 1 a CTA has two accumulators and works on
// the next tile while the epilogue reads the last one out.  With MT = 2 a tile is 256 x BN: both
// accumulators belong to one tile, every row of B that comes into shared memory is used twice,
// and a product whose 128-row tiles would need a second, partly empty round over the SMs has
// half as many tiles (the epilogue then runs after the products, not beside them).
template <int BN, int STAGES, bool OUT_F32, bool SILU, int MT = 1>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_bf16_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                            const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    constexpr uint32_t A_SUB = BM * BK * 2, A_BYTES = MT * A_SUB, B_BYTES = BN * BK * 2;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "the epilogue reads 32 columns at a time");
    static_assert(MT == 1 || MT == 2, "one or two 128-row blocks per tile");
    constexpr int NACC = MT == 1 ? 2 : 1;                       // accumulators of MT x BN columns
    constexpr uint32_t TMEM_COLS = 2 * BN <= 256 ? 256 : 512;   // 2 x BN columns in use; powers of two only
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint64_t* bars = (uint64_t*)(smem + STAGES * (A_BYTES + B_BYTES));
    uint64_t* full = bars;                       // [STAGES]
    uint64_t* empty = bars + STAGES;             // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;      // [2] an accumulator is complete
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2] the epilogue has read it out
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_a = (p.rows_a + MT * BM - 1) / (MT * BM), tiles_b = (p.rows_b + BN - 1) / BN;
    const int num_tiles = tiles_a * tiles_b;
    const int num_kb = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);           // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        pdl_wait();                                          // the activations come from the kernel before
        int it = 0;                                          // k-blocks issued so far, over all tiles
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int a0 = (tile % tiles_a) * (MT * BM), b0 = (tile / tiles_a) * BN;
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag)) goto done;
                const uint32_t bar = smem_u32(&full[s]);
                mbar_expect_tx(bar, A_BYTES + B_BYTES);
                // (a block of rows past the end of A arrives as zeros and counts its bytes all the same)
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    tma_load_2d(smem_u32(smem_a + s * A_BYTES + m * A_SUB), &map_a, bar, kb * BK, a0 + m * BM);
                tma_load_2d(smem_u32(smem_b + s * B_BYTES), &map_b, bar, kb * BK, b0);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = instr_desc_bf16(BN);
        int it = 0, local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int acc = local % NACC;
            // the epilogue must have emptied this accumulator (NACC tiles ago)
            if (!mbar_wait(smem_u32(&acc_empty[acc]), ((local / NACC) & 1) ^ 1, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + (uint32_t)(acc * MT * BN);
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&full[s]), (it / STAGES) & 1, abort_flag)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t db = smem_desc_sw128(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint64_t da = smem_desc_sw128(smem_u32(smem_a + s * A_BYTES + m * A_SUB));
                        umma_bf16(tmem_d + (uint32_t)(m * BN), da + 2 * kk, db + 2 * kk, idesc,
                                  (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(&empty[s]));
            }
            umma_commit(smem_u32(&acc_full[acc]));
        }
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int acc = local % NACC;
            const int a0 = (tile % tiles_a) * (MT * BM), b0 = (tile / tiles_a) * BN;
            if (!mbar_wait(smem_u32(&acc_full[acc]), (local / NACC) & 1, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < MT * BN; c += 32) {
                const int m = c / BN, c0 = c - m * BN;       // BN is a multiple of 32: no chunk spans two blocks
                const int a = a0 + m * BM + quarter * 32 + lane;
                const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * MT * BN);
                uint32_t r[32];
                tmem_ld32(trow + (uint32_t)c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (a >= p.rows_a) continue;
                const int b_first = b0 + c0;
                if (b_first >= p.rows_b) continue;
                store_chunk32<OUT_F32, SILU>(p, r, a, b_first);
            }
            // this warp is done with the accumulator: let the MMA warp reuse it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
        }
    }
done:
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicOr(p.err, CRANE_ERR_WAIT_TIMEOUT);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Many tokens, two SMs per tile (tcgen05 cta_group::2).
//
// A cluster of two CTAs computes a 256 x BN tile: each CTA loads its own 128 rows of A and only
// HALF of the tile's rows of B; the MMA, issued by the first CTA of the pair for both, reads A
// and B from the shared memory of both SMs and leaves each CTA's 128 rows of the accumulator in
// that CTA's tensor memory.  Per k-block a CTA thus takes in 16 KB + BN / 2 x 128 bytes instead
// of 16 KB + BN x 128 bytes, which is what the single-CTA kernel above is bound by.
//
// Barriers: the stage-full barriers that count live in the first CTA (the peer's copies signal
// them through the cta_group::2 form of the TMA load); stage-empty and accumulator-full are
// signalled in both CTAs by one multicast commit; accumulator-empty lives in the first CTA and
// takes the arrivals of the epilogue warps of both.  Every wait is bounded as above.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// dst in this CTA, the barrier (a shared::cluster address) in either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                               uint32_t accumulate) {
    const uint32_t z = 0;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(z)
        : "memory");
}
// arrives on the barrier at this shared-memory offset in every CTA of `mask`
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_bar, uint32_t rank) {
    asm volatile(
        "{\n"
        ".reg .b32 remote;\n"
        "mapa.shared::cluster.u32 remote, %0, %1;\n"
        "mbarrier.arrive.shared::cluster.b64 _, [remote];\n"
        "}\n" ::"r"(local_bar), "r"(rank)
        : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

//
// MT = 2: the pair's tile is 512 x BN, two 256-row blocks one under the other, each CTA holding two
// accumulators of BN columns (rows 0..127 / 128..255 of either block).  A CTA then takes in 32 KB of
// A and BN / 2 rows of B per k-block for twice the products, the least operand traffic per product
// of all the kernels here; with more than 256 accumulator columns per tile there is no second
// accumulator to work into while the epilogue reads, so the epilogue of a tile is not hidden.
template <int BN, int STAGES, bool SILU, int MT = 1>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const GemmParams p) {
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "BN / 2 rows of B per CTA, 32 columns per epilogue step");
    static_assert(MT == 1 || MT == 2, "one or two 256-row blocks per tile");
    constexpr int BH = BN / 2;                                   // rows of B that one CTA loads
    constexpr uint32_t A_SUB = BM * BK * 2, A_BYTES = MT * A_SUB, B_BYTES = BH * BK * 2;
    constexpr int NACC = 2 * MT * BN <= 512 ? 2 : 1;             // accumulators of MT x BN columns
    constexpr uint32_t TMEM_COLS = NACC * MT * BN <= 256 ? 256 : 512;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // both CTAs of a pair round up by the same amount, so offsets match across them
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint64_t* bars = (uint64_t*)(smem + STAGES * (A_BYTES + B_BYTES));
    uint64_t* full = bars;                       // [STAGES] used in the first CTA only
    uint64_t* empty = bars + STAGES;             // [STAGES] in both
    uint64_t* acc_full = bars + 2 * STAGES;      // [2] in both
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2] used in the first CTA only
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                     // 0: issues the MMAs
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    constexpr int TILE_ROWS = 2 * BM * MT;
    const int tiles_a = (p.rows_a + TILE_ROWS - 1) / TILE_ROWS, tiles_b = (p.rows_b + BN - 1) / BN;
    const int num_tiles = tiles_a * tiles_b;
    const int num_kb = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 8);               // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // the same warp of both CTAs, the same slot offset
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                          // the peer's barriers exist before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        pdl_wait();
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            const int a0 = (tile % tiles_a) * TILE_ROWS + (int)rank * BM;
            const int b0 = (tile / tiles_a) * BN + (int)rank * BH;
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag)) goto done;
                const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
                if (rank == 0) mbar_expect_tx(smem_u32(&full[s]), 2 * (A_BYTES + B_BYTES));   // both CTAs' bytes
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    tma_load_2d_pair(smem_u32(smem_a + s * A_BYTES + m * A_SUB), &map_a, bar, kb * BK,
                                     a0 + m * 2 * BM);
                tma_load_2d_pair(smem_u32(smem_b + s * B_BYTES), &map_b, bar, kb * BK, b0);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------- MMA issuer (first CTA, for the pair) ----------------
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                               ((uint32_t)((2 * BM) >> 4) << 24);
        int it = 0, local = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
            const int acc = local % NACC;
            if (!mbar_wait(smem_u32(&acc_empty[acc]), ((local / NACC) & 1) ^ 1, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + (uint32_t)(acc * MT * BN);
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&full[s]), (it / STAGES) & 1, abort_flag)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t db = smem_desc_sw128(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint64_t da = smem_desc_sw128(smem_u32(smem_a + s * A_BYTES + m * A_SUB));
                        umma_bf16_pair(tmem_d + (uint32_t)(m * BN), da + 2 * kk, db + 2 * kk, idesc,
                                       (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                umma_commit_pair(smem_u32(&empty[s]), 3);        // the stage is free in both CTAs
            }
            umma_commit_pair(smem_u32(&acc_full[acc]), 3);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue (both CTAs, each its 128 rows) ----------------
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
            const int acc = local % NACC;
            const int a0 = (tile % tiles_a) * TILE_ROWS + (int)rank * BM, b0 = (tile / tiles_a) * BN;
            if (!mbar_wait(smem_u32(&acc_full[acc]), (local / NACC) & 1, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * MT * BN);
#pragma unroll 1
            for (int c = 0; c < MT * BN; c += 32) {
                const int m = c / BN, c0 = c - m * BN;           // BN is a multiple of 32: no chunk spans two blocks
                const int a = a0 + m * 2 * BM + quarter * 32 + lane;
                uint32_t r[32];
                tmem_ld32(trow + (uint32_t)c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (a >= p.rows_a) continue;
                const int b_first = b0 + c0;
                if (b_first >= p.rows_b) continue;
                store_chunk32<false, SILU>(p, r, a, b_first);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(smem_u32(&acc_empty[acc]), 0);
        }
    }
done:
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicOr(p.err, CRANE_ERR_WAIT_TIMEOUT);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();                          // neither CTA frees tensor memory the other's MMA may touch
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (EncodeTiledFn)sym;
    }
    return fn;
}

// [rows, k] bf16, k contiguous, `ld` elements between rows; box of 64 x box_rows.
// A descriptor depends on nothing but these arguments, and a model asks for the same few
// hundred (every weight, a handful of activation buffers) step after step: the last ones are
// kept per thread and found again by their arguments, which saves the driver call.
struct MapSlot {
    const void* ptr;
    long long ld;
    int rows, k, box_rows;
    bool used;
    CUtensorMap map;
};
constexpr int MAP_SLOTS = 1024;                      // a power of two

bool make_map(CUtensorMap* map, const void* ptr, int rows, int k, long long ld, int box_rows) {
    static thread_local MapSlot* slots = nullptr;
    if (!slots) slots = new MapSlot[MAP_SLOTS]();
    uint64_t h = (uint64_t)(uintptr_t)ptr >> 4;
    h ^= ((uint64_t)(uint32_t)rows << 20) ^ ((uint64_t)(uint32_t)box_rows << 44) ^ ((uint64_t)(uint32_t)k << 8);
    h *= 0x9E3779B97F4A7C15ull;
    MapSlot& sl = slots[(h >> 40) & (MAP_SLOTS - 1)];
    if (sl.used && sl.ptr == ptr && sl.rows == rows && sl.k == k && sl.ld == ld && sl.box_rows == box_rows) {
        *map = sl.map;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    sl.ptr = ptr; sl.ld = ld; sl.rows = rows; sl.k = k; sl.box_rows = box_rows; sl.map = *map; sl.used = true;
    return true;
}

template <int BN, int STAGES, bool OUT_F32, bool TRANSPOSED>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid,
           cudaStream_t st) {
    constexpr size_t smem = STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
    auto kern = gemm_bf16_kernel<BN, STAGES, OUT_F32, TRANSPOSED>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return crane_launch(kern, grid, dim3(NUM_THREADS), smem, st, ma, mb, p);
}

template <int BN, int STAGES, bool OUT_F32, bool SILU = false, int MT = 1>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int num_tiles,
                      cudaStream_t st) {
    constexpr size_t smem = STAGES * (MT * BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
    static_assert(smem <= 232448, "more shared memory than a CTA can have");
    auto kern = gemm_bf16_persistent_kernel<BN, STAGES, OUT_F32, SILU, MT>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int ctas = num_tiles < sms ? num_tiles : sms;
    return crane_launch(kern, dim3(ctas), dim3(NUM_THREADS), smem, st, ma, mb, p);
}

template <int BN, int STAGES, bool SILU, int MT = 1>
int launch_pair(const void* A, const void* B, int rows_a, int rows_b, int k, long long lda, long long ldb,
                const GemmParams& p, cudaStream_t st) {
    constexpr size_t smem = STAGES * (MT * BM * BK * 2 + (BN / 2) * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
    static_assert(smem <= 232448, "more shared memory than a CTA can have");
    auto kern = gemm_bf16_pair_kernel<BN, STAGES, SILU, MT>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    CUtensorMap ma, mb;
    if (!make_map(&ma, A, rows_a, k, lda, BM) || !make_map(&mb, B, rows_b, k, ldb, BN / 2))
        return (int)cudaErrorInvalidValue;
    const int tiles = ((rows_a + 2 * BM * MT - 1) / (2 * BM * MT)) * ((rows_b + BN - 1) / BN);
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    return crane_launch_cluster(kern, dim3(2 * pairs), dim3(NUM_THREADS), smem, dim3(2, 1, 1), st, ma, mb, p);
}

template <bool OUT_F32, bool TRANSPOSED>
int dispatch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid,
                cudaStream_t st) {
    switch (bn) {
        // the narrow tiles keep their shared memory under half an SM's, so that the CTAs of
        // the next product can move in beside them and request their weights early
        case 16: return launch<16, 6, OUT_F32, TRANSPOSED>(ma, mb, p, grid, st);
        case 32: return launch<32, 5, OUT_F32, TRANSPOSED>(ma, mb, p, grid, st);
        case 64: return launch<64, 4, OUT_F32, TRANSPOSED>(ma, mb, p, grid, st);
        case 128: return launch<128, 6, OUT_F32, TRANSPOSED>(ma, mb, p, grid, st);
        case 256: return launch<256, 4, OUT_F32, TRANSPOSED>(ma, mb, p, grid, st);
    }
    return (int)cudaErrorInvalidValue;
}

}  // namespace

// D[a, b] = sum_k A[a, k] B[b, k].  bn: columns (rows of B) per tile, 16..256.
// tile_rows: 128, or 256 (bf16 output, untransposed, no slices, no epilogue, bn 128 / 192 / 256 only).
// epilogue: 0 none, 1 silu(gate) * up (see the persistent kernel).
// out_f32 / transposed as in the kernel; split_k > 1 writes float partial sums
// [split_k][...] into `out` (which must then be float) `split_stride` apart.
// Requirements (checked, cudaErrorInvalidValue otherwise): k % 8 == 0, lda and
// ldb multiples of 8 elements, A and B 16-byte aligned.
CRANE_API int crane_gemm_bf16_tcgen05(const void* A, const void* B, const float* bias, void* out,
                                      int rows_a, int rows_b, int k, long long lda, long long ldb,
                                      long long ld_out, int bn, int tile_rows, int out_f32, int transposed,
                                      int split_k, long long split_stride, int epilogue,
                                      const void* prefetch, long long prefetch_bytes, int* err,
                                      cudaStream_t st) {
    if (rows_a <= 0 || rows_b <= 0) return 0;
    if (k <= 0 || (k & 7) || (lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15))
        return (int)cudaErrorInvalidValue;
    if (split_k < 1) split_k = 1;
    if (split_k > 1 && !out_f32) return (int)cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    if (!make_map(&ma, A, rows_a, k, lda, BM) || !make_map(&mb, B, rows_b, k, ldb, bn))
        return (int)cudaErrorInvalidValue;
    const int num_kb = (k + BK - 1) / BK;
    if (split_k > num_kb) split_k = num_kb;
    GemmParams p;
    p.rows_a = rows_a; p.rows_b = rows_b; p.k = k;
    p.out = out; p.ld_out = ld_out; p.split_stride = split_stride; p.bias = bias; p.err = err;
    p.prefetch = ((uintptr_t)prefetch & 15) ? nullptr : (const uint8_t*)prefetch;   // (only the narrow-tile kernel asks)
    p.prefetch_bytes = prefetch_bytes > 0 ? prefetch_bytes : 0;
    dim3 grid((rows_a + BM - 1) / BM, (rows_b + bn - 1) / bn, split_k);
    if (tile_rows == 2 * BM) {
        if (transposed || split_k != 1 || out_f32 || epilogue != 0) return (int)cudaErrorInvalidValue;
        const int tiles = (int)(((rows_a + 2 * BM - 1) / (2 * BM)) * grid.y);
        switch (bn) {
            case 128: return launch_persistent<128, 4, false, false, 2>(ma, mb, p, tiles, st);
            case 192: return launch_persistent<192, 4, false, false, 2>(ma, mb, p, tiles, st);
            case 256: return launch_persistent<256, 3, false, false, 2>(ma, mb, p, tiles, st);
        }
        return (int)cudaErrorInvalidValue;
    }
    if (tile_rows != BM) return (int)cudaErrorInvalidValue;
    if (epilogue == 1) {
        // silu(gate) * up: bf16 output of rows_b / 2 columns; the weights' rows in blocks of 16 + 16
        if (transposed || split_k != 1 || out_f32 || bias != nullptr || (rows_b & 31) || (ld_out & 7) ||
            ((uintptr_t)out & 15))
            return (int)cudaErrorInvalidValue;
        const int tiles = (int)(grid.x * grid.y);
        switch (bn) {
            case 128: return launch_persistent<128, 6, false, true>(ma, mb, p, tiles, st);
            case 160: return launch_persistent<160, 6, false, true>(ma, mb, p, tiles, st);
            case 192: return launch_persistent<192, 5, false, true>(ma, mb, p, tiles, st);
            case 224: return launch_persistent<224, 5, false, true>(ma, mb, p, tiles, st);
            case 256: return launch_persistent<256, 4, false, true>(ma, mb, p, tiles, st);
        }
        return (int)cudaErrorInvalidValue;
    }
    if (epilogue != 0) return (int)cudaErrorInvalidValue;
    if (!transposed && split_k == 1 && !out_f32 && (bn == 160 || bn == 192 || bn == 224)) {
        // widths between 128 and 256: chosen when they fill the last wave of tiles better
        const int tiles = (int)(grid.x * grid.y);
        if (bn == 160) return launch_persistent<160, 6, false>(ma, mb, p, tiles, st);
        if (bn == 192) return launch_persistent<192, 5, false>(ma, mb, p, tiles, st);
        return launch_persistent<224, 5, false>(ma, mb, p, tiles, st);
    }
    if (!transposed && split_k == 1 && (bn == 128 || bn == 256)) {
        const int tiles = (int)(grid.x * grid.y);
        if (bn == 256)
            return out_f32 ? launch_persistent<256, 4, true>(ma, mb, p, tiles, st)
                           : launch_persistent<256, 4, false>(ma, mb, p, tiles, st);
        return out_f32 ? launch_persistent<128, 6, true>(ma, mb, p, tiles, st)
                       : launch_persistent<128, 6, false>(ma, mb, p, tiles, st);
    }
    if (out_f32)
        return transposed ? dispatch_bn<true, true>(bn, ma, mb, p, grid, st)
                          : dispatch_bn<true, false>(bn, ma, mb, p, grid, st);
    return transposed ? dispatch_bn<false, true>(bn, ma, mb, p, grid, st)
                      : dispatch_bn<false, false>(bn, ma, mb, p, grid, st);
}

// The same product as crane_gemm_bf16_tcgen05 for many tokens (bf16 output, untransposed, no
// slices) on pairs of SMs: 256 x bn tiles, bn in 128, 192, 224, 256, or (tile_rows 512) 512 x bn
// tiles, bn in 192, 224, 256.  epilogue as there.
CRANE_API int crane_gemm_bf16_pair(const void* A, const void* B, const float* bias, void* out, int rows_a,
                                   int rows_b, int k, long long lda, long long ldb, long long ld_out,
                                   int bn, int tile_rows, int epilogue, int* err, cudaStream_t st) {
    if (rows_a <= 0 || rows_b <= 0) return 0;
    if (k <= 0 || (k & 7) || (lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15))
        return (int)cudaErrorInvalidValue;
    if (tile_rows != 2 * BM && tile_rows != 4 * BM) return (int)cudaErrorInvalidValue;
    const bool tall = tile_rows == 4 * BM;                  // 512-row tiles: bn 192, 224 or 256
    GemmParams p;
    p.rows_a = rows_a; p.rows_b = rows_b; p.k = k;
    p.out = out; p.ld_out = ld_out; p.split_stride = 0; p.bias = bias; p.err = err;
    p.prefetch = nullptr; p.prefetch_bytes = 0;
    if (epilogue == 1) {
        if (bias != nullptr || (rows_b & 31) || (ld_out & 7) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
        if (tall) switch (bn) {
            case 192: return launch_pair<192, 5, true, 2>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
            case 224: return launch_pair<224, 4, true, 2>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
            case 256: return launch_pair<256, 4, true, 2>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
            default: return (int)cudaErrorInvalidValue;
        }
        switch (bn) {
            case 128: return launch_pair<128, 8, true>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
            case 192: return launch_pair<192, 7, true>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
            case 224: return launch_pair<224, 6, true>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
            case 256: return launch_pair<256, 6, true>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        }
        return (int)cudaErrorInvalidValue;
    }
    if (epilogue != 0) return (int)cudaErrorInvalidValue;
    if (tall) switch (bn) {
        case 192: return launch_pair<192, 5, false, 2>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        case 224: return launch_pair<224, 4, false, 2>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        case 256: return launch_pair<256, 4, false, 2>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        default: return (int)cudaErrorInvalidValue;
    }
    switch (bn) {
        case 128: return launch_pair<128, 8, false>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        case 192: return launch_pair<192, 7, false>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        case 224: return launch_pair<224, 6, false>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
        case 256: return launch_pair<256, 6, false>(A, B, rows_a, rows_b, k, lda, ldb, p, st);
    }
    return (int)cudaErrorInvalidValue;
}
