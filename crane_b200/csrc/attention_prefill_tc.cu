// Flash attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bf16, pages of 16 tokens or a larger power of two).  One CTA owns 128 query rows
// of one request and one query head and walks over the keys in tiles of 128:
//
//   warp 0 (all lanes)    TMA: the Q tile once, then K and V tiles from the
//                         paged pool, page by page through the block table,
//                         into 128-byte-swizzled shared memory (two stages);
//                         every lane looks one page up and issues one copy;
//   warp 1 (one thread)   tcgen05.mma:  S = Q K^T  (float, tensor memory, two
//                         buffers);
//   last warp (one thread) tcgen05.mma:  O += P V  (float, tensor memory), P
//                         read from tensor memory as the A operand;
//   the warps between     two threads per query row, each with half of the
//                         tile's keys and half of O's columns: read S with
//                         tcgen05.ld, scale, mask (causal + window), running
//                         max (agreed through shared memory) and sum,
//                         P = exp2(S - max) as bf16 pairs into one of two P
//                         buffers in tensor memory; rescale O in tensor memory
//                         when the running max has moved far; at the end
//                         O / sum -> out.
//
// How it got this shape (per-role clock stamps of one CTA showed what a tile
// waits for; leaving work out one piece at a time had shown nothing, because
// several chains were about equally long): one producer lane issuing all
// copies took longer per tile than anything else; then one thread issuing
// both products; the softmax arithmetic was never the longest chain.
//
// A row keeps the maximum it uses for its exponentials until a later score
// exceeds it by more than 2^8; until then P simply carries the factor (at most
// 256, exact in float and in range for bf16), and O is rescaled only on those
// rare moves.  The result is the same softmax (scores = q k^T / sqrt(d), causal,
// query head h reads kv head h / (nq / nkv): crane-core/src/models/
// hunyuan_dense/modeling.rs:611-636, 1012-1033).
//
// Every mbarrier wait is bounded; on a timeout the kernel records
// CRANE_ERR_WAIT_TIMEOUT, every role leaves its loop, tensor memory is freed.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int D = 128;            // head size
constexpr int BQ = 128;           // query rows per CTA = MMA M
constexpr int BKV = 128;          // keys per tile
constexpr int SPLIT = 2;              // softmax threads per query row (4 measured no faster)
constexpr int SM_WARPS = 4 * SPLIT;   // softmax warps
constexpr int PV_WARP = 2 + SM_WARPS; // warp 0: TMA, warp 1: first product, then the softmax warps, then the second product
constexpr int NUM_THREADS = 32 * (PV_WARP + 1);
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr uint32_t HALF_BYTES = 128 * 128;          // 128 rows x 64 bf16: one swizzled half tile
constexpr uint32_t TILE_BYTES = 2 * HALF_BYTES;     // 128 x 128 bf16
constexpr float RESCALE_THRESHOLD = 8.0f;           // in log2 units

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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// K-major operand (rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand: rows are positions along K (keys), each row holds 64
// consecutive MN elements (128 bytes, swizzled); the next 64 MN elements are one
// half tile further (leading byte offset), the next 8 rows 1024 bytes further
// (stride byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(HALF_BYTES >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, bf16 x bf16 -> f32, M = 128, N = 128; b_mn: B operand MN-major
__device__ __forceinline__ uint32_t idesc(bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t id, uint32_t acc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"(acc)
        : "memory");
}
// the same with the A operand in tensor memory (16-bit elements, two per column)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t id, uint32_t acc) {
    const uint32_t z = 0;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(id), "r"(acc), "r"(z)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
          "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
          "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
          "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
          "r"(r[15])
        : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t* r) {
    static_assert(N == 16 || N == 32, "16 or 32 columns");
    if (N == 32) tmem_st32(taddr, r);
    else tmem_st16(taddr, r);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Params {
    __nv_bfloat16* out;          // [N, nq * D]
    const int* cu_q;
    const int* kv_len;
    const int* block_table;
    int max_blocks, num_pages, page_size, n_entries, nq, nkv, window;
    int skip_single;             // entries of one token have no tile here (the decode kernel takes them)
    float scale_log2;
    int* err;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sm_q = smem;                          // [2 halves][128][128 B]
    uint8_t* sm_k = sm_q + TILE_BYTES;             // [2 stages][2 halves][128][128 B]
    uint8_t* sm_v = sm_k + 2 * TILE_BYTES;         // [2 stages][2 halves (of d)][128 keys][128 B]
    uint64_t* bars = (uint64_t*)(sm_v + 2 * TILE_BYTES);
    uint64_t* q_full = bars;            // Q has landed
    uint64_t* k_full = bars + 1;        // [2]
    uint64_t* v_full = bars + 3;        // [2]
    uint64_t* k_empty = bars + 5;       // [2] the S product that read the stage is done
    uint64_t* v_empty = bars + 7;       // [2] the O product that read the stage is done
    uint64_t* s_full = bars + 9;        // [2] S is complete in tensor memory
    uint64_t* s_empty = bars + 11;      // [2] the softmax threads have read S out
    uint64_t* p_full = bars + 13;       // [2] P is in its tensor-memory buffer (and O rescaled if need be)
    uint64_t* pv_done = bars + 15;      // [2] the O product that read the P buffer is done
    uint32_t* tmem_slot = (uint32_t*)(bars + 17);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* sm_x = (float*)(bars + 18);             // [2 tiles in turn][SPLIT][128 rows]: what the threads
                                                   // of a row tell each other (maximum, sum)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which request and which of its query tiles (a request's last tiles, which read the most
    // keys, come first)
    // CTAs are handed to the SMs in the order of their index, heads fastest: all heads of a request's
    // last query tile (which reads the most keys) first, its first tile's last.  SMs that finish a
    // short tile early then pick up what is left of the long work, and heads of one kv head read the
    // same K and V tiles at about the same time.
    int e = 0, tile = blockIdx.y;
    for (; e < p.n_entries; ++e) {
        const int rows = p.cu_q[e + 1] - p.cu_q[e];
        const int tiles = (p.skip_single && rows == 1) ? 0 : (rows + BQ - 1) / BQ;
        if (tile < tiles) {
            tile = tiles - 1 - tile;
            break;
        }
        tile -= tiles;
    }
    const bool active = e < p.n_entries;
    const int h = blockIdx.x, g = active ? h / (p.nq / p.nkv) : 0;
    const int row0 = active ? p.cu_q[e] : 0, q_len = active ? p.cu_q[e + 1] - row0 : 0;
    const int pos0 = active ? p.kv_len[e] - q_len : 0;
    const int r_begin = tile * BQ, r_end = min(q_len, r_begin + BQ);
    const int p_first = pos0 + r_begin, p_last = pos0 + r_end - 1;
    const int lo = (p.window > 0 && p_first - p.window + 1 > 0) ? p_first - p.window + 1 : 0;
    const int t_begin = lo / BKV, t_end = active ? p_last / BKV + 1 : 0;
    const int n_tiles = max(0, t_end - t_begin);
    const int* table = p.block_table + (long long)e * p.max_blocks;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), SM_WARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&p_full[b]), SM_WARPS);
            mbar_init(smem_u32(&pv_done[b]), 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // S buffers at columns 0 and 128, O at 256, two P buffers (bf16 pairs: 64 columns each) at 384 and 448.
    // P stays in tensor memory and is the A operand of the second product from there: it never goes
    // through shared memory, whose bandwidth the products' operand reads and the copies already fill.
    const uint32_t tmem_o = tmem_base + 256, tmem_p = tmem_base + 384;
    pdl_launch_dependents();

    if (warp == 0 && n_tiles > 0) {
        // ---------------- TMA: the whole warp ----------------
        // A tile of K and a tile of V are 2 x (pages per tile) x 2 halves copies, at most 32: every
        // lane looks its page number up and issues its one copy, so that the look-ups and the
        // issue of the copies take the time of one, not of all in a row (one lane doing them all
        // took longer per tile than the softmax or the products).
        pdl_wait();
        if (lane == 0) {
            mbar_expect_tx(smem_u32(q_full), TILE_BYTES);
            tma_load_2d(smem_u32(sm_q), &map_q, smem_u32(q_full), h * D, row0 + r_begin);
            tma_load_2d(smem_u32(sm_q + HALF_BYTES), &map_q, smem_u32(q_full), h * D + 64, row0 + r_begin);
        }
        const int ps = p.page_size;                    // 16, 32, 64, 128 or a larger power of two
        const int shift = 31 - __clz(ps);
        const int chunks = ps < BKV ? BKV >> shift : 1;   // pages per tile: 8, 4, 2 or 1 (or a tile is part of a page)
        const int piece = ps < BKV ? ps : BKV;         // keys per copy
        const int per_kv = 2 * chunks;                 // copies per tile of K (or V)
        const bool worker = lane < 2 * per_kv;
        const int my_kv = lane / per_kv, c = (lane % per_kv) >> 1, hf = lane & 1;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            const uint32_t parity = ((j >> 1) & 1) ^ 1;
            // a page that lies wholly after the last key is read as the last valid one: its keys
            // are masked, only the byte count has to be complete (likewise a page wholly before
            // the window's first key)
            int blk = (((t_begin + j) * BKV) >> shift) + c;
            blk = max(lo >> shift, min(blk, p_last >> shift));
            int page = worker ? table[blk] : 0;
            if (page < 0 || page >= p.num_pages) {
                atomicOr(p.err, CRANE_ERR_PAGE_RANGE);
                page = 0;
            }
            const int row = ((page * p.nkv + g) << shift) + (ps > BKV ? ((t_begin + j) * BKV) & (ps - 1) : 0);
            for (int kv = 0; kv < 2; ++kv) {
                uint64_t* full = kv ? &v_full[s] : &k_full[s];
                uint64_t* empty = kv ? &v_empty[s] : &k_empty[s];
                uint8_t* dst = (kv ? sm_v : sm_k) + s * TILE_BYTES;
                if (!mbar_wait(smem_u32(empty), parity, abort_flag)) goto done;
                if (lane == 0) mbar_expect_tx(smem_u32(full), TILE_BYTES);
                __syncwarp();
                if (worker && my_kv == kv)
                    tma_load_2d(smem_u32(dst + hf * HALF_BYTES + c * piece * 128), kv ? &map_v : &map_k,
                                smem_u32(full), hf * 64, row);
            }
        }
    } else if (warp == 1 && lane == 0 && n_tiles > 0) {
        // ---------------- first product: S_j = Q K_j^T into S buffer j & 1 ----------------
        // The two products are issued by a thread each: one thread's waits and issue slots for
        // both were the longest chain of a tile; tcgen05.commit counts the issuing thread's MMAs.
        const uint32_t id_s = idesc(false);
        // Operand descriptors are made once; a step along the tile only adds to the address field
        // (16-byte units, the whole of shared memory fits its 14 bits).
        const uint64_t dq = desc_kmajor(smem_u32(sm_q)), dk = desc_kmajor(smem_u32(sm_k));
        if (!mbar_wait(smem_u32(q_full), 0, abort_flag)) goto done;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            if (!mbar_wait(smem_u32(&k_full[s]), (j >> 1) & 1, abort_flag)) goto done;
            if (!mbar_wait(smem_u32(&s_empty[s]), ((j >> 1) & 1) ^ 1, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t dks = dk + (uint64_t)(s * (TILE_BYTES >> 4));
            const uint32_t ts = tmem_base + s * 128;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t off = (uint64_t)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4);
                umma(ts, dq + off, dks + off, id_s, kk > 0);
            }
            umma_commit(smem_u32(&s_full[s]));
            umma_commit(smem_u32(&k_empty[s]));
        }
    } else if (warp == PV_WARP && lane == 0 && n_tiles > 0) {
        // ---------------- second product: O += P_j V_j, P from tensor memory ----------------
        const uint32_t id_o = idesc(true);
        const uint64_t dv = desc_mnmajor(smem_u32(sm_v));
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            if (!mbar_wait(smem_u32(&v_full[s]), (j >> 1) & 1, abort_flag)) goto done;
            if (!mbar_wait(smem_u32(&p_full[s]), (j >> 1) & 1, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t dvs = dv + (uint64_t)(s * (TILE_BYTES >> 4));
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
                // P: 16 keys further along K = 8 columns; V: 16 keys further = 16 rows = 2048 bytes
                umma_ts(tmem_o, tmem_p + s * 64 + kk * 8, dvs + (uint64_t)(kk * (2048 >> 4)), id_o, (j > 0 || kk > 0));
            }
            umma_commit(smem_u32(&pv_done[s]));
            umma_commit(smem_u32(&v_empty[s]));
        }
    } else if (warp >= 2 && warp < PV_WARP && n_tiles > 0) {
        // ---------------- softmax, correction, epilogue: SPLIT threads per query row ----------------
        // Warps w, w + 4, w + 8, ... own the same 32 rows (a warp reaches the lanes of tensor memory
        // given by its index modulo 4); each takes its share of every tile's keys and of O's columns.
        // They agree on the row's maximum through shared memory once per tile and keep a partial sum
        // each.  That gives every scheduler several softmax warps to alternate between and shortens
        // the chain of exponentials and conversions per tile.
        constexpr int HK = BKV / SPLIT;
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                   // which share: 0 .. SPLIT - 1
        const int r = quarter * 32 + lane;                  // row of the tile = lane of tensor memory
        const int pos = pos0 + r_begin + r;                 // this row's position
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int pair_bar = 1 + quarter;                   // named barrier of the warps of these rows
        float m_ref = -INFINITY, l = 0.f;                   // maximum in use, running sum of this half
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            if (!mbar_wait(smem_u32(&s_full[s]), (j >> 1) & 1, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int tile_base = (t_begin + j) * BKV;
            const int key_base = tile_base + half * HK;     // first key of this thread's half
            // this half of the row of scores into registers, then the buffer is free for the next S
            uint32_t v[HK];
#pragma unroll
            for (int c0 = 0; c0 < HK; c0 += 32) tmem_ld32(tmem_base + lane_addr + s * 128 + half * HK + c0, v + c0);
            static_assert(HK % 32 == 0, "a softmax thread reads its scores 32 columns at a time");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_empty[s]));
            // only tiles that touch the diagonal or the window's edge need the mask
            const bool need_mask = tile_base + BKV - 1 > p_first || tile_base < lo ||
                                   (p.window > 0 && tile_base <= p_last - p.window);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < HK; ++i) {
                    const int key = key_base + i;
                    const bool ok = key <= pos && (p.window <= 0 || key > pos - p.window);
                    if (!ok) v[i] = 0xff800000u;            // -inf
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < HK; i += 4) {
                mx0 = fmaxf(mx0, __uint_as_float(v[i]));
                mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(v[i + 2]));
                mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
            }
            // the row's maximum over both halves
            float* xch = sm_x + (j & 1) * SPLIT * BQ;
            float mine = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            xch[half * BQ + r] = mine;
            asm volatile("bar.sync %0, %1;" ::"r"(pair_bar), "n"(32 * SPLIT) : "memory");
#pragma unroll
            for (int o = 0; o < SPLIT; ++o) mine = fmaxf(mine, xch[o * BQ + r]);
            const float mx = mine * p.scale_log2;           // scale > 0
            // keep the maximum in use unless the row moved far above it (decided per warp, because
            // the tensor-memory accesses below are warp-wide; both warps of a row decide alike)
            const bool far = mx > m_ref + RESCALE_THRESHOLD;
            const bool warp_far = __any_sync(0xffffffffu, far);
            float factor = 1.f;
            if (far) {
                factor = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - mx);
                m_ref = mx;
            }
            // P = exp2(S * scale - m_ref), bf16 pairs, still in registers
            const float nbase = (m_ref == -INFINITY) ? 0.f : -m_ref;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int i = 0; i < HK; i += 4) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, nbase));
                const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, nbase));
                const float p2 = fast_exp2(fmaf(__uint_as_float(v[i + 2]), p.scale_log2, nbase));
                const float p3 = fast_exp2(fmaf(__uint_as_float(v[i + 3]), p.scale_log2, nbase));
                s0 += p0; s1 += p1; s2 += p2; s3 += p3;
                __nv_bfloat162 b0 = __floats2bfloat162_rn(p0, p1), b1 = __floats2bfloat162_rn(p2, p3);
                v[i >> 1] = *(uint32_t*)&b0;                 // the first half of v now holds the packed pairs
                v[(i >> 1) + 1] = *(uint32_t*)&b1;
            }
            l = l * factor + ((s0 + s1) + (s2 + s3));
            // P has two buffers: this tile's P may be written while the O product of the tile before
            // still reads the other one; only the product two tiles back must be done.  O can be
            // rescaled only when the product of the tile before is done, which is waited for just then.
            if (j > 1 && !mbar_wait(smem_u32(&pv_done[s]), ((j >> 1) & 1) ^ 1, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (warp_far && j > 0) {
                if (!mbar_wait(smem_u32(&pv_done[s ^ 1]), ((j - 1) >> 1) & 1, abort_flag)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // this thread's half of the row of O
#pragma unroll 1
                for (int c0 = half * (D / SPLIT); c0 < (half + 1) * (D / SPLIT); c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + lane_addr + c0, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tmem_st32(tmem_o + lane_addr + c0, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // this half's 64 keys, two to a column, into the tile's P buffer in tensor memory
            tmem_st_n<HK / 2>(tmem_p + lane_addr + s * 64 + half * (HK / 2), v);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            // P and O are ready for the second product
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[s]));
        }
        // ---- epilogue: O / l, this thread's half of the columns; l is the sum of both halves ----
        if (!mbar_wait(smem_u32(&pv_done[(n_tiles - 1) & 1]), ((n_tiles - 1) >> 1) & 1, abort_flag)) goto done;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
            float* xch = sm_x + (n_tiles & 1) * SPLIT * BQ;
            xch[half * BQ + r] = l;
            asm volatile("bar.sync %0, %1;" ::"r"(pair_bar), "n"(32 * SPLIT) : "memory");
            l = 0.f;
#pragma unroll
            for (int o = 0; o < SPLIT; ++o) l += xch[o * BQ + r];            // the same order for every thread
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool store = r_begin + r < r_end;
        __nv_bfloat16* orow = p.out + ((long long)(row0 + r_begin + r) * p.nq + h) * D;
#pragma unroll 1
        for (int c0 = half * (D / SPLIT); c0 < (half + 1) * (D / SPLIT); c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_addr + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (store) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 w;
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                    __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                    __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                    w.x = *(uint32_t*)&b0; w.y = *(uint32_t*)&b1; w.z = *(uint32_t*)&b2; w.w = *(uint32_t*)&b3;
                    *(uint4*)(orow + c0 + i) = w;
                }
            }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// The same attention with TWO query heads of one kv head per CTA (the heads
// 2y and 2y + 1 of head pair y = blockIdx.y; the group size nq / nkv must be
// even).  Both heads have the same rows and therefore the same key tiles, so
//   * every K and V tile that comes into shared memory serves two heads: half
//     the traffic from L2 per product, which is what bounds the one-head kernel
//     once a prompt's keys no longer stay close to the SMs;
//   * the two heads take turns on the tensor cores: while one head's softmax
//     threads work on their scores, the other head's products run.
// Tensor memory: S of head A at columns 0..127, S of head B at 128..255, O of A
// at 256..383, O of B at 384..511.  P (bf16 pairs, 64 columns) is written over
// the first half of its head's S, from where the second product reads it.
// One thread issues all products, in this order (j: key tile):
//   S_A(0) S_B(0) | PV_A(j) S_A(j+1) PV_B(j) S_B(j+1) | ...
// The tensor cores run products in the order of issue, so S_x(j+1) overwrites
// P_x(j) only after PV_x(j) has read it, and a completed S_x(j) tells head x's
// softmax threads that PV_x(j-1) is complete as well (O_x may be rescaled).
// One softmax thread per query row and head: warps 4..7 head A, warps 8..11
// head B (a warp reaches the 32 lanes of tensor memory given by its index
// modulo 4).  They hold a whole row of 128 scores in registers, for which the
// two softmax warpgroups take registers over from the first one (setmaxnreg).
constexpr int PAIR_THREADS = 384;

__global__ void __launch_bounds__(PAIR_THREADS, 1)
prefill_attn_tc_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sm_q = smem;                          // [2 heads][2 halves][128][128 B]
    uint8_t* sm_k = sm_q + 2 * TILE_BYTES;         // [2 stages][2 halves][128][128 B]
    uint8_t* sm_v = sm_k + 2 * TILE_BYTES;         // [2 stages][2 halves (of d)][128 keys][128 B]
    uint64_t* bars = (uint64_t*)(sm_v + 2 * TILE_BYTES);
    uint64_t* q_full = bars;            // both heads' Q have landed
    uint64_t* k_full = bars + 1;        // [2]
    uint64_t* v_full = bars + 3;        // [2]
    uint64_t* k_empty = bars + 5;       // [2] both heads' S products that read the stage are done
    uint64_t* v_empty = bars + 7;       // [2] both heads' O products that read the stage are done
    uint64_t* s_full = bars + 9;        // [2 heads] S of the head's next tile is complete
    uint64_t* p_full = bars + 11;       // [2 heads] the head's P is in tensor memory (O rescaled if need be)
    uint64_t* o_done = bars + 13;       // every product is complete
    uint32_t* tmem_slot = (uint32_t*)(bars + 14);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int e = 0, tile = blockIdx.y;                  // head pairs fastest, as in the one-head kernel
    for (; e < p.n_entries; ++e) {
        const int rows = p.cu_q[e + 1] - p.cu_q[e];
        const int tiles = (p.skip_single && rows == 1) ? 0 : (rows + BQ - 1) / BQ;
        if (tile < tiles) {
            tile = tiles - 1 - tile;
            break;
        }
        tile -= tiles;
    }
    const bool active = e < p.n_entries;
    const int h_a = 2 * blockIdx.x, g = active ? h_a / (p.nq / p.nkv) : 0;
    const int row0 = active ? p.cu_q[e] : 0, q_len = active ? p.cu_q[e + 1] - row0 : 0;
    const int pos0 = active ? p.kv_len[e] - q_len : 0;
    const int r_begin = tile * BQ, r_end = min(q_len, r_begin + BQ);
    const int p_first = pos0 + r_begin, p_last = pos0 + r_end - 1;
    const int lo = (p.window > 0 && p_first - p.window + 1 > 0) ? p_first - p.window + 1 : 0;
    const int t_begin = lo / BKV, t_end = active ? p_last / BKV + 1 : 0;
    const int n_tiles = max(0, t_end - t_begin);
    const int* table = p.block_table + (long long)e * p.max_blocks;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&p_full[s]), 4);          // the four warps of a head's softmax warpgroup
        }
        mbar_init(smem_u32(o_done), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp < 4) {
        // the copying and the issuing warps need few registers: the softmax warpgroups take the rest
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        if (warp == 0 && n_tiles > 0) {
            // ---------------- TMA: the whole warp (as in the one-head kernel) ----------------
            pdl_wait();
            if (lane == 0) {
                mbar_expect_tx(smem_u32(q_full), 2 * TILE_BYTES);
                for (int x = 0; x < 2; ++x) {
                    tma_load_2d(smem_u32(sm_q + x * TILE_BYTES), &map_q, smem_u32(q_full), (h_a + x) * D,
                                row0 + r_begin);
                    tma_load_2d(smem_u32(sm_q + x * TILE_BYTES + HALF_BYTES), &map_q, smem_u32(q_full),
                                (h_a + x) * D + 64, row0 + r_begin);
                }
            }
            const int ps = p.page_size;                    // 16, 32, 64, 128 or a larger power of two
            const int shift = 31 - __clz(ps);
            const int chunks = ps < BKV ? BKV >> shift : 1;   // pages per tile: 8, 4, 2 or 1 (or a tile is part of a page)
            const int piece = ps < BKV ? ps : BKV;         // keys per copy
            const int per_kv = 2 * chunks;                 // copies per tile of K (or V)
            const bool worker = lane < 2 * per_kv;
            const int my_kv = lane / per_kv, c = (lane % per_kv) >> 1, hf = lane & 1;
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t parity = ((j >> 1) & 1) ^ 1;
                int blk = (((t_begin + j) * BKV) >> shift) + c;
                blk = max(lo >> shift, min(blk, p_last >> shift));
                int page = worker ? table[blk] : 0;
                if (page < 0 || page >= p.num_pages) {
                    atomicOr(p.err, CRANE_ERR_PAGE_RANGE);
                    page = 0;
                }
                const int row = ((page * p.nkv + g) << shift) + (ps > BKV ? ((t_begin + j) * BKV) & (ps - 1) : 0);
                for (int kv = 0; kv < 2; ++kv) {
                    uint64_t* full = kv ? &v_full[s] : &k_full[s];
                    uint64_t* empty = kv ? &v_empty[s] : &k_empty[s];
                    uint8_t* dst = (kv ? sm_v : sm_k) + s * TILE_BYTES;
                    if (!mbar_wait(smem_u32(empty), parity, abort_flag)) goto done;
                    if (lane == 0) mbar_expect_tx(smem_u32(full), TILE_BYTES);
                    __syncwarp();
                    if (worker && my_kv == kv)
                        tma_load_2d(smem_u32(dst + hf * HALF_BYTES + c * piece * 128), kv ? &map_v : &map_k,
                                    smem_u32(full), hf * 64, row);
                }
            }
        } else if (warp == 1 && lane == 0 && n_tiles > 0) {
            // ---------------- all products, one thread ----------------
            const uint32_t id_s = idesc(false), id_o = idesc(true);
            const uint64_t dq = desc_kmajor(smem_u32(sm_q)), dk = desc_kmajor(smem_u32(sm_k));
            const uint64_t dv = desc_mnmajor(smem_u32(sm_v));
            auto issue_s = [&](int x, int stage) {              // S_x = Q_x K^T
                const uint64_t dqx = dq + (uint64_t)(x * (TILE_BYTES >> 4)), dks = dk + (uint64_t)(stage * (TILE_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4);
                    umma(tmem_base + x * 128, dqx + off, dks + off, id_s, kk > 0);
                }
                umma_commit(smem_u32(&s_full[x]));
            };
            auto issue_pv = [&](int x, int stage, bool first) {  // O_x += P_x V, P_x from tensor memory
                const uint64_t dvs = dv + (uint64_t)(stage * (TILE_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk)
                    umma_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + kk * 8, dvs + (uint64_t)(kk * (2048 >> 4)),
                            id_o, (!first || kk > 0));
            };
            if (!mbar_wait(smem_u32(q_full), 0, abort_flag)) goto done;
            if (!mbar_wait(smem_u32(&k_full[0]), 0, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(0, 0);
            issue_s(1, 0);
            umma_commit(smem_u32(&k_empty[0]));
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const bool more = j + 1 < n_tiles;
                if (!mbar_wait(smem_u32(&v_full[s]), (j >> 1) & 1, abort_flag)) goto done;
                if (!mbar_wait(smem_u32(&p_full[0]), j & 1, abort_flag)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_pv(0, s, j == 0);
                if (more) {
                    if (!mbar_wait(smem_u32(&k_full[s ^ 1]), ((j + 1) >> 1) & 1, abort_flag)) goto done;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(0, s ^ 1);
                }
                if (!mbar_wait(smem_u32(&p_full[1]), j & 1, abort_flag)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_pv(1, s, j == 0);
                umma_commit(smem_u32(&v_empty[s]));
                if (more) {
                    issue_s(1, s ^ 1);
                    umma_commit(smem_u32(&k_empty[s ^ 1]));
                }
            }
            umma_commit(smem_u32(o_done));
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        if (n_tiles > 0) {
            // ---------------- softmax, correction, epilogue: one thread per query row and head ----------------
            const int x = (warp >> 2) - 1;                      // 0: head A, 1: head B
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;                  // row of the tile = lane of tensor memory
            const int pos = pos0 + r_begin + r;                 // this row's position
            const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
            const uint32_t tmem_s = tmem_base + x * 128 + lane_addr;
            const uint32_t tmem_ox = tmem_base + 256 + x * 128 + lane_addr;
            float m_ref = -INFINITY, l = 0.f;                   // maximum in use, running sum
            for (int j = 0; j < n_tiles; ++j) {
                if (!mbar_wait(smem_u32(&s_full[x]), j & 1, abort_flag)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int tile_base = (t_begin + j) * BKV;
                uint32_t v[BKV];
#pragma unroll
                for (int c0 = 0; c0 < BKV; c0 += 32) tmem_ld32(tmem_s + c0, v + c0);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const bool need_mask = tile_base + BKV - 1 > p_first || tile_base < lo ||
                                       (p.window > 0 && tile_base <= p_last - p.window);
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < BKV; ++i) {
                        const int key = tile_base + i;
                        const bool ok = key <= pos && (p.window <= 0 || key > pos - p.window);
                        if (!ok) v[i] = 0xff800000u;            // -inf
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < BKV; i += 4) {
                    mx0 = fmaxf(mx0, __uint_as_float(v[i]));
                    mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(v[i + 2]));
                    mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;    // scale > 0
                const bool far = mx > m_ref + RESCALE_THRESHOLD;
                const bool warp_far = __any_sync(0xffffffffu, far);
                float factor = 1.f;
                if (far) {
                    factor = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - mx);
                    m_ref = mx;
                }
                const float nbase = (m_ref == -INFINITY) ? 0.f : -m_ref;
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int i = 0; i < BKV; i += 4) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, nbase));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, nbase));
                    const float p2 = fast_exp2(fmaf(__uint_as_float(v[i + 2]), p.scale_log2, nbase));
                    const float p3 = fast_exp2(fmaf(__uint_as_float(v[i + 3]), p.scale_log2, nbase));
                    s0 += p0; s1 += p1; s2 += p2; s3 += p3;
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(p0, p1), b1 = __floats2bfloat162_rn(p2, p3);
                    v[i >> 1] = *(uint32_t*)&b0;                 // the first half of v now holds the packed pairs
                    v[(i >> 1) + 1] = *(uint32_t*)&b1;
                }
                l = l * factor + ((s0 + s1) + (s2 + s3));
                if (warp_far && j > 0) {
                    // the head's O product of the tile before is complete (its S product was issued behind it)
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem_ox + c0, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                        tmem_st32(tmem_ox + c0, o);
                    }
                }
                // the row's 128 keys, two to a column, over the first half of the head's S
                tmem_st32(tmem_s, v);
                tmem_st32(tmem_s + 32, v + 32);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&p_full[x]));
            }
            // ---- epilogue: O / l ----
            if (!mbar_wait(smem_u32(o_done), 0, abort_flag)) goto done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool store = r_begin + r < r_end;
            __nv_bfloat16* orow = p.out + ((long long)(row0 + r_begin + r) * p.nq + h_a + x) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_ox + c0, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (store) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                        __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        w.x = *(uint32_t*)&b0; w.y = *(uint32_t*)&b1; w.z = *(uint32_t*)&b2; w.w = *(uint32_t*)&b3;
                        *(uint4*)(orow + c0 + i) = w;
                    }
                }
            }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                     : "memory");
    }
}

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
// CRANE_PREFILL_PAIR=0 keeps the kernel of one head per CTA for every shape, =2 takes the kernel of
// two heads per CTA wherever the group size allows it (for measuring one against the other).
int pair_kernel_mode() {
    static int mode = -1;
    if (mode < 0) {
        const char* v = getenv("CRANE_PREFILL_PAIR");
        mode = v == nullptr ? 1 : (v[0] == '0' ? 0 : (v[0] == '2' ? 2 : 1));
    }
    return mode;
}
// [rows, cols] bf16, cols contiguous; box of 64 columns x box_rows rows, 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

CRANE_API int crane_prefill_attention_tc_supports(int d, int nq, int nkv, int page_size) {
    if (nkv <= 0 || nq % nkv != 0) return 0;
    // pages of 16 to 128 tokens (a 128-key tile is 8 to 1 of them) or larger powers of two (a tile is part of one)
    return d == 128 && page_size >= 16 && (page_size & (page_size - 1)) == 0;
}

// total_q_tiles: sum over the entries of ceil(q_len / 128) (or more).  q is [n_tokens, nq * 128].
// skip_single != 0: entries of exactly one token are left out and count no tile.
CRANE_API int crane_prefill_attention_tc(const void* q, void* out, const void* k_pool, const void* v_pool,
                                         const int* cu_q, const int* kv_len, const int* block_table,
                                         int max_blocks, int num_pages, int page_size, int n_entries,
                                         int n_tokens, int total_q_tiles, int nq, int nkv, int d, int window,
                                         float scale, int skip_single, int* err, cudaStream_t st) {
    if (n_entries <= 0 || total_q_tiles <= 0) return 0;
    if (!crane_prefill_attention_tc_supports(d, nq, nkv, page_size)) return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mk, mv;
    const long long pool_rows = (long long)num_pages * nkv * page_size;
    if (!make_map(&mq, q, n_tokens, (long long)nq * D, BQ) || !make_map(&mk, k_pool, pool_rows, D, page_size < BKV ? page_size : BKV) ||
        !make_map(&mv, v_pool, pool_rows, D, page_size < BKV ? page_size : BKV))
        return (int)cudaErrorInvalidValue;
    Params p;
    p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.kv_len = kv_len; p.block_table = block_table;
    p.max_blocks = max_blocks; p.num_pages = num_pages; p.page_size = page_size; p.n_entries = n_entries;
    p.nq = nq; p.nkv = nkv; p.window = window; p.skip_single = skip_single; p.scale_log2 = scale * 1.4426950408889634f; p.err = err;
    // Two heads of a kv head per CTA (every K and V tile serves both, the heads take turns on the
    // tensor cores) where there are CTAs enough to keep every SM busy to the end even so.  Measured
    // at 16 / 4 heads, one head against two per CTA: a whole prompt of 4,096 tokens 88 against 78 us, of
    // 8,192 the same (265 us, 0.63 of the bf16 peak), 2,048 rows behind 30,000 cached keys 562 against
    // 519 us; below that the coarser grain loses (2,048 tokens 29 against 44 us; 512 rows behind 8,192
    // keys, 64 CTAs against 32, 81 against 143 us).
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int pair_mode = pair_kernel_mode();
    if ((nq / nkv) % 2 == 0 && (pair_mode == 2 || (pair_mode == 1 && 10LL * total_q_tiles * (nq / 2) >= 17LL * sms))) {
        constexpr size_t pair_smem = 6 * TILE_BYTES + 14 * 8 + 16 + 1024;
        static bool pair_configured = false;
        if (!pair_configured) {
            if (cudaFuncSetAttribute(prefill_attn_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)pair_smem) != cudaSuccess)
                return (int)cudaGetLastError();
            pair_configured = true;
        }
        return crane_launch(prefill_attn_tc_pair_kernel, dim3(nq / 2, total_q_tiles), dim3(PAIR_THREADS), pair_smem,
                            st, mq, mk, mv, p);
    }
    constexpr size_t smem = 5 * TILE_BYTES + 18 * 8 + 2 * SPLIT * BQ * 4 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return crane_launch(prefill_attn_tc_kernel, dim3(nq, total_q_tiles), dim3(NUM_THREADS), smem, st, mq, mk,
                        mv, p);
}
