// Warp-level pieces shared by the bf16 attention kernels: tensor-core tiles
// (mma.sync m16n8k16, float accumulate), ldmatrix loads from padded shared
// memory rows, 16-byte asynchronous copies with zero fill.
//
// These kernels read each key and value once per group of query heads and are
// bound by memory traffic, which the warp-level MMA keeps up with; the dense
// products of the model run on tcgen05 (gemm_tcgen05.cu).
#pragma once
#include "common.cuh"

namespace attn {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
// 16 bytes global -> shared; bytes == 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// c += a (16x16, row) * b (16x8, col), bf16 in, float out
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// A tile of TILE key (or value) rows of D bf16 in shared memory; rows are
// 2*D + 16 bytes apart, which spreads the 8 rows of an ldmatrix over the banks.
template <int D>
struct Tile {
    static constexpr int ROW_BYTES = 2 * D + 16;
    static constexpr int CHUNKS = D / 8;          // 16-byte pieces per row
};

// Copies rows [key0, key0 + ROWS) of one kv head from the paged pool into a
// tile, by THREADS threads together, asynchronously.  Rows outside [lo, hi] and rows whose page
// number is out of range become zeros (the latter is also reported).
template <int D, int ROWS, int THREADS = 32>
__device__ __forceinline__ void load_tile_async(uint32_t tile, const __nv_bfloat16* pool,
                                                const int* table, int num_pages, int page_size,
                                                int nkv, int g, int key0, int lo, int hi, int lane,
                                                bool& bad_page) {
    // `lane` is the thread's index among the THREADS that copy the tile together
    constexpr int CH = Tile<D>::CHUNKS;
    static_assert(ROWS * CH % THREADS == 0, "the tile must divide among the copying threads");
    if (page_size % ROWS == 0) {
        // tiles start at multiples of ROWS, so the whole tile lies in one page: one look-up
        const bool wanted = key0 <= hi && key0 + ROWS - 1 >= lo;
        const __nv_bfloat16* base = pool;
        bool ok = false;
        if (wanted) {
            const int page = table[key0 / page_size];
            ok = page >= 0 && page < num_pages;
            if (!ok) bad_page = true;
            else base = pool + (((long long)page * nkv + g) * page_size + key0 % page_size) * D;
        }
#pragma unroll
        for (int i = 0; i < ROWS * CH / THREADS; ++i) {
            const int c = i * THREADS + lane;
            const int row = c / CH, col = c % CH;
            const int j = key0 + row;
            const bool in = ok && j >= lo && j <= hi;
            cp_async16(tile + row * Tile<D>::ROW_BYTES + col * 16,
                       in ? base + row * D + col * 8 : pool, in ? 16 : 0);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < ROWS * CH / THREADS; ++i) {
        const int c = i * THREADS + lane;
        const int row = c / CH, col = c % CH;
        const int j = key0 + row;
        const __nv_bfloat16* src = pool;
        int bytes = 0;
        if (j >= lo && j <= hi) {
            const int page = table[j / page_size];
            if (page >= 0 && page < num_pages) {
                src = pool + (((long long)page * nkv + g) * page_size + j % page_size) * D + col * 8;
                bytes = 16;
            } else {
                bad_page = true;
            }
        }
        cp_async16(tile + row * Tile<D>::ROW_BYTES + col * 16, src, bytes);
    }
}

}  // namespace attn
