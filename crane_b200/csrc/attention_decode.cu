// Attention of single decoded tokens over the paged cache (bf16), split along
// the keys.  One CTA takes one (slice of the keys, kv head, request); its
// warps take 32-key tiles of the slice in turn (each warp with its own ring of
// three tile stages fed by cp.async), each keeping its own running softmax, and
// merge at the end.  All query heads that share the kv head ride
// in the rows of one MMA tile, so every key and value is read once per group
// (the reference's decode path groups the same way:
// crane-core/src/models/hunyuan_dense/modeling.rs:575-608).  With more than one
// slice the CTAs leave (max, sum, unnormalised output) per slice in scratch
// memory and a second kernel merges the slices.
//
// scores = q k^T / sqrt(d), softmax in float, keys lo..pos of the request with
// lo = max(0, pos - window + 1) (modeling.rs:579-601).
//
// At head size 128 with pages of a multiple of 32 tokens the tiles come by TMA
// instead (paged_decode_attn_tma_kernel below): one lane asks for a whole tile
// with four bulk tensor copies and the warp waits on an mbarrier, which takes
// the per-row address arithmetic and the 32 cp.async per lane and tile out of
// the instruction stream that bounds this kernel at small batches.
#include <cuda.h>

#include "attention_mma.cuh"
#include "no_alloc.h"

namespace {
using namespace attn;

constexpr int TILE = 32;
constexpr int WARPS = 2;         // 2 warps x 3 stages: 104 KB at head size 128, two CTAs (or a product's CTA) per SM
constexpr int NSTAGE = 3;        // tiles of K and V per warp in shared memory: one in use, two on the way

// The fused form takes the step's q, k and v raw from the product that made
// them and does, inside the attention kernel, what rope_norm_cache_kernel does
// for a decode step: rotary encoding, per-head RMSNorm, and the write of the new
// key and value into their page (crane-core/src/models/hunyuan_dense/
// modeling.rs:541-557).  Every CTA prepares the query rows of its group itself;
// the warp whose tile holds the new position prepares the new key and value,
// puts them into its tile in shared memory and into the page.
struct FusedArgs {
    const __nv_bfloat16* qkv;       // rows [q | k | v] of the step's tokens, or null when they
    const float* qkv_parts;         // come as float partial sums [part][row][col]
    int n_parts;
    long long part_stride;
    int qkv_stride;
    int has_kv;                     // 0: the layer reads another layer's cache and writes nothing
    int rotary;
    const float* cos_tab;
    const float* sin_tab;
    int table_len;
    const float* q_norm_w;          // [D] or null
    const float* k_norm_w;
    float eps;
    __nv_bfloat16* k_pool_w;        // the pools again, writable
    __nv_bfloat16* v_pool_w;
    RopeParams rope;                // pairing, rotated width, norm order, norm weight offset
    int general;                    // 0: the defaults (whole head, contiguous halves, norm after, plain w)
};

// A single element of the raw product (see raw2 for pairs).
__device__ __forceinline__ float raw1(const FusedArgs& a, long long idx) {
    if (a.qkv_parts == nullptr) return __bfloat162float(a.qkv[idx]);
    float s = 0.f;
    for (int i = 0; i < a.n_parts; ++i) s += a.qkv_parts[(long long)i * a.part_stride + idx];
    return __bfloat162float(__float2bfloat16_rn(s));
}

__device__ __forceinline__ float2 raw2(const FusedArgs& a, long long idx) {
    if (a.qkv_parts == nullptr) return __bfloat1622float2(*(const __nv_bfloat162*)(a.qkv + idx));
    float2 s = make_float2(0.f, 0.f);
    for (int i = 0; i < a.n_parts; i += 8) {                 // eight loads in flight, added in slice order
        float2 p[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            p[j] = (i + j < a.n_parts) ? *(const float2*)(a.qkv_parts + (long long)(i + j) * a.part_stride + idx)
                                       : make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s.x += p[j].x;
            s.y += p[j].y;
        }
    }
    // rounded once to bf16, like a product that was written out whole
    return __bfloat1622float2(__floats2bfloat162_rn(s.x, s.y));
}

// One head row of D elements at `src`: rotary encoding at position pos, then
// RMSNorm with weight nw (if any); lane owns the neighbours j, j + 1 and their
// partners in the second half.  Results (rounded to bf16) go to dst0 and, if
// given, dst1.
template <int D, bool GENERAL>
__device__ __forceinline__ void rope_norm_row(const FusedArgs& a, long long src, int pos, bool rotate,
                                              const float* nw, int lane, __nv_bfloat16* dst0,
                                              __nv_bfloat16* dst1) {
    if (GENERAL) {
        rope_norm_general<(D / 2 + 31) / 32>(a.rope, D, pos, rotate, a.cos_tab, a.sin_tab, nw, a.eps, lane,
                                             [&](int e) { return raw1(a, src + e); },
                                             [&](int e, float v) {
                                                 const __nv_bfloat16 b = __float2bfloat16_rn(v);
                                                 dst0[e] = b;
                                                 if (dst1 != nullptr) dst1[e] = b;
                                             });
        return;
    }
    constexpr int HALF = D / 2;
    constexpr int IT = (HALF + 63) / 64;
    float2 x1[IT], x2[IT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < IT; ++i) {
        const int j = 2 * lane + 64 * i;
        x1[i] = x2[i] = make_float2(0.f, 0.f);
        if (j < HALF) {
            const float2 u = raw2(a, src + j), v = raw2(a, src + j + HALF);
            if (rotate) {
                const float2 c = *(const float2*)(a.cos_tab + (long long)pos * HALF + j);
                const float2 sn = *(const float2*)(a.sin_tab + (long long)pos * HALF + j);
                x1[i] = make_float2(u.x * c.x - v.x * sn.x, u.y * c.y - v.y * sn.y);
                x2[i] = make_float2(v.x * c.x + u.x * sn.x, v.y * c.y + u.y * sn.y);
            } else {
                x1[i] = u;
                x2[i] = v;
            }
            ss += x1[i].x * x1[i].x + x1[i].y * x1[i].y + x2[i].x * x2[i].x + x2[i].y * x2[i].y;
        }
    }
    float rstd = 1.f;
    if (nw != nullptr) rstd = rsqrtf(warp_sum(ss) / (float)D + a.eps);
#pragma unroll
    for (int i = 0; i < IT; ++i) {
        const int j = 2 * lane + 64 * i;
        if (j < HALF) {
            float2 y1 = x1[i], y2 = x2[i];
            if (nw != nullptr) {
                const float2 w1 = *(const float2*)(nw + j), w2 = *(const float2*)(nw + j + HALF);
                y1 = make_float2(y1.x * rstd * w1.x, y1.y * rstd * w1.y);
                y2 = make_float2(y2.x * rstd * w2.x, y2.y * rstd * w2.y);
            }
            const __nv_bfloat162 b1 = __floats2bfloat162_rn(y1.x, y1.y), b2 = __floats2bfloat162_rn(y2.x, y2.y);
            *(__nv_bfloat162*)(dst0 + j) = b1;
            *(__nv_bfloat162*)(dst0 + j + HALF) = b2;
            if (dst1 != nullptr) {
                *(__nv_bfloat162*)(dst1 + j) = b1;
                *(__nv_bfloat162*)(dst1 + j + HALF) = b2;
            }
        }
    }
}

// Up to four pairs of neighbours of the raw product at once: from partial sums, the loads of
// all four places and of up to eight slices are in flight together (one round trip instead of
// one per place), added in slice order and rounded once as in raw2.
__device__ __forceinline__ void raw2x4(const FusedArgs& a, const long long (&idx)[4], int n, float2 (&out)[4]) {
    if (a.qkv_parts == nullptr) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            out[q] = q < n ? __bfloat1622float2(*(const __nv_bfloat162*)(a.qkv + idx[q])) : make_float2(0.f, 0.f);
        return;
    }
    float2 acc[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[q] = make_float2(0.f, 0.f);
    for (int i = 0; i < a.n_parts; i += 8) {
        float2 p[4][8];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                p[q][j] = (q < n && i + j < a.n_parts)
                              ? *(const float2*)(a.qkv_parts + (long long)(i + j) * a.part_stride + idx[q])
                              : make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[q].x += p[q][j].x;
                acc[q].y += p[q][j].y;
            }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) out[q] = __bfloat1622float2(__floats2bfloat162_rn(acc[q].x, acc[q].y));
}

// The same in two phases, so that the loads of several rows (and of the tables,
// which are the same for all rows of a position) are in flight together.
template <int D>
struct RowRegs {
    static constexpr int IT = (D / 2 + 63) / 64;
    float2 u[IT], v[IT];
};
template <int D>
__device__ __forceinline__ void row_load(const FusedArgs& a, long long src, int lane, RowRegs<D>& r) {
#pragma unroll
    for (int i = 0; i < RowRegs<D>::IT; ++i) {
        const int j = 2 * lane + 64 * i;
        r.u[i] = r.v[i] = make_float2(0.f, 0.f);
        if (j < D / 2) {
            r.u[i] = raw2(a, src + j);
            r.v[i] = raw2(a, src + j + D / 2);
        }
    }
}
// cs/sn: this lane's cosines and sines (read when `rotate`), w1/w2: its norm weights (read when `norm`).
template <int D>
__device__ __forceinline__ void row_finish(const RowRegs<D>& r, bool rotate, const float2* cs, const float2* sn,
                                           bool norm, const float2* w1, const float2* w2, float eps, int lane,
                                           __nv_bfloat16* dst0, __nv_bfloat16* dst1) {
    constexpr int IT = RowRegs<D>::IT;
    float2 x1[IT], x2[IT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < IT; ++i) {
        const float2 u = r.u[i], v = r.v[i];
        if (rotate) {
            x1[i] = make_float2(u.x * cs[i].x - v.x * sn[i].x, u.y * cs[i].y - v.y * sn[i].y);
            x2[i] = make_float2(v.x * cs[i].x + u.x * sn[i].x, v.y * cs[i].y + u.y * sn[i].y);
        } else {
            x1[i] = u;
            x2[i] = v;
        }
        ss += x1[i].x * x1[i].x + x1[i].y * x1[i].y + x2[i].x * x2[i].x + x2[i].y * x2[i].y;
    }
    float rstd = 1.f;
    if (norm) rstd = rsqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
    for (int i = 0; i < IT; ++i) {
        const int j = 2 * lane + 64 * i;
        if (j < D / 2) {
            float2 y1 = x1[i], y2 = x2[i];
            if (norm) {
                y1 = make_float2(y1.x * rstd * w1[i].x, y1.y * rstd * w1[i].y);
                y2 = make_float2(y2.x * rstd * w2[i].x, y2.y * rstd * w2[i].y);
            }
            const __nv_bfloat162 b1 = __floats2bfloat162_rn(y1.x, y1.y), b2 = __floats2bfloat162_rn(y2.x, y2.y);
            *(__nv_bfloat162*)(dst0 + j) = b1;
            *(__nv_bfloat162*)(dst0 + j + D / 2) = b2;
            if (dst1 != nullptr) {
                *(__nv_bfloat162*)(dst1 + j) = b1;
                *(__nv_bfloat162*)(dst1 + j + D / 2) = b2;
            }
        }
    }
}

// GENERAL: the instantiation for heads rotated or normalised otherwise than by the defaults (FusedArgs::
// rope); it is a kernel of its own so that the serving kernel carries none of its code.
template <int D, bool FUSED, bool GENERAL>
__global__ void __launch_bounds__(WARPS * 32)
paged_decode_attn_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                         float* __restrict__ part_o, float* __restrict__ part_ml,
                         const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_len, const int* __restrict__ block_table,
                         int max_blocks, int num_pages, int page_size, int nq, int nkv, int window,
                         float scale_log2, int n_splits, int* err, const FusedArgs fa) {
    constexpr int RB = Tile<D>::ROW_BYTES;
    constexpr int TILE_BYTES = TILE * RB;
    constexpr int KS = D / 16;                     // k-steps of q k^T
    constexpr int DN = D / 8;                      // n-tiles of the output
    extern __shared__ __align__(16) uint8_t smem[];

    pdl_launch_dependents();
    // Keys and values of earlier positions were written by earlier steps; when this kernel makes
    // the new position's row itself (fused, own cache) it can request its first tiles before the
    // kernel that produces q, k and v has finished.  Otherwise everything waits for that kernel.
    const bool early = FUSED && fa.has_kv != 0;
    if (!early) pdl_wait();
    const int split = blockIdx.x, g = blockIdx.y, e = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_rep = nq / nkv;
    const int t = cu_q[e];
    // an entry with a prompt portion (or a padding entry without rows) is another kernel's: all
    // CTAs of the entry, which are all CTAs of its cluster, leave here
    if (cu_q[e + 1] - t != 1) return;
    const int pos = kv_len[e] - 1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (long long)e * max_blocks;

    const int first_tile = lo / TILE;
    const int n_tiles = pos / TILE - first_tile + 1;
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int tile_begin = first_tile + split * per_split;
    const int tile_end = min(first_tile + n_tiles, tile_begin + per_split);

    // this warp's ring of (K tile, V tile) stages
    const uint32_t wbase = smem_u32(smem) + warp * NSTAGE * 2 * TILE_BYTES;

    bool bad_page = false;
    // keys that are read from the pages: the new position's row is made here when fused
    const bool makes_kv = FUSED && fa.has_kv != 0;
    const int hi = makes_kv ? pos - 1 : pos;
    float o[DN][4];
#pragma unroll
    for (int i = 0; i < DN; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    int ti = tile_begin + warp;
#pragma unroll
    for (int s = 0; s < NSTAGE - 1; ++s) {
        const int tj = ti + s * WARPS;
        if (tj < tile_end) {
            const uint32_t st = wbase + s * 2 * TILE_BYTES;
            load_tile_async<D, TILE>(st, k_pool, table, num_pages, page_size, nkv, g, tj * TILE, lo,
                                     hi, lane, bad_page);
            load_tile_async<D, TILE>(st + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g,
                                     tj * TILE, lo, hi, lane, bad_page);
        }
        cp_async_commit();
    }
    if (early) pdl_wait();                         // from here on q, k and v of this step are read
    // query rows: row r of the MMA tile is query head g * n_rep + r
    uint32_t qf[KS][4];
    bool rotate = FUSED && fa.rotary != 0;
    if (FUSED) {
        if (rotate && (pos < 0 || pos >= fa.table_len)) {
            if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_POSITION_RANGE);
            rotate = false;
        }
        // the group's query rows, encoded and normalised here, staged in shared memory
        __nv_bfloat16* q_s = (__nv_bfloat16*)(smem + WARPS * NSTAGE * 2 * TILE_BYTES);   // [16][D]
        for (int i = threadIdx.x; i < 16 * D / 2; i += WARPS * 32) ((uint32_t*)q_s)[i] = 0u;
        __syncthreads();
        for (int r = warp; r < n_rep; r += WARPS)
            rope_norm_row<D, GENERAL>(fa, (long long)t * fa.qkv_stride + (long long)(g * n_rep + r) * D, pos, rotate,
                                      fa.q_norm_w, lane, q_s + r * D, nullptr);
        __syncthreads();
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                qf[ks][i] = *(const uint32_t*)(q_s + (r0 + (i & 1) * 8) * D + ks * 16 + c0 + (i >> 1) * 8);
    } else {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = r0 + (i & 1) * 8, c = ks * 16 + c0 + (i >> 1) * 8;
                uint32_t v = 0;
                if (r < n_rep)
                    v = *(const uint32_t*)(q + ((long long)t * nq + g * n_rep + r) * D + c);
                qf[ks][i] = v;
            }
        }
    }
    for (int it = 0; ti < tile_end; ti += WARPS, ++it) {
        const uint32_t kt = wbase + (it % NSTAGE) * 2 * TILE_BYTES, vt = kt + TILE_BYTES;
        const int nxt = ti + (NSTAGE - 1) * WARPS;
        if (nxt < tile_end) {
            // the stage that the previous iteration finished with
            const uint32_t nk = wbase + ((it + NSTAGE - 1) % NSTAGE) * 2 * TILE_BYTES;
            load_tile_async<D, TILE>(nk, k_pool, table, num_pages, page_size, nkv, g, nxt * TILE, lo,
                                     hi, lane, bad_page);
            load_tile_async<D, TILE>(nk + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g,
                                     nxt * TILE, lo, hi, lane, bad_page);
        }
        cp_async_commit();
        cp_async_wait<NSTAGE - 1>();
        __syncwarp();
        if (makes_kv && ti == pos / TILE) {
            // this tile holds the new position: its key (encoded, normalised) and value are
            // made here, for the tile in shared memory and for the page
            const int page = table[pos / page_size];
            if (page < 0 || page >= num_pages) {
                bad_page = true;
            } else {
                const long long prow = (((long long)page * nkv + g) * page_size + pos % page_size) * D;
                uint8_t* stage = smem + (size_t)(warp * NSTAGE + it % NSTAGE) * 2 * TILE_BYTES;
                __nv_bfloat16* k_row = (__nv_bfloat16*)(stage + (pos % TILE) * RB);
                __nv_bfloat16* v_row = (__nv_bfloat16*)(stage + TILE_BYTES + (pos % TILE) * RB);
                const long long row_src = (long long)t * fa.qkv_stride;
                rope_norm_row<D, GENERAL>(fa, row_src + (long long)(nq + g) * D, pos, rotate, fa.k_norm_w, lane, k_row,
                                          fa.k_pool_w + prow);
                for (int c = 2 * lane; c < D; c += 64) {
                    const float2 x = raw2(fa, row_src + (long long)(nq + nkv + g) * D + c);
                    const __nv_bfloat162 b = __floats2bfloat162_rn(x.x, x.y);
                    *(__nv_bfloat162*)(v_row + c) = b;
                    *(__nv_bfloat162*)(fa.v_pool_w + prow + c) = b;
                }
            }
            __syncwarp();
        }

        // ---- scores: 16 rows x 32 keys ----
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                // matrices: (keys +0..7, d lo), (keys +0..7, d hi), (keys +8..15, d lo), (keys +8..15, d hi)
                const int key = half * 16 + (mi >> 1) * 8 + mr;
                const int chunk = ks * 2 + (mi & 1);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kt + key * RB + chunk * 16, b0, b1, b2, b3);
                mma_bf16(s[half * 2], qf[ks], b0, b1);
                mma_bf16(s[half * 2 + 1], qf[ks], b2, b3);
            }
        }
        // ---- mask, running softmax ----
        const int key0 = ti * TILE + (lane & 3) * 2;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = key0 + nt * 8 + (c & 1);
                const float v = (j >= lo && j <= pos) ? s[nt][c] * scale_log2 : -INFINITY;
                s[nt][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        float corr[2], base[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float m_new = fmaxf(m[h], quad_max(mx[h]));
            base[h] = (m_new == -INFINITY) ? 0.f : m_new;
            corr[h] = exp2f(m[h] - base[h]);           // exp2(-inf) = 0 on the first tile
            m[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = exp2f(s[nt][c] - base[c >> 1]);
                s[nt][c] = p;
                rs[c >> 1] += p;
            }
        l[0] = l[0] * corr[0] + rs[0];
        l[1] = l[1] * corr[1] + rs[1];
#pragma unroll
        for (int i = 0; i < DN; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // ---- output += p v ----
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dn = 0; dn < DN; dn += 2) {
                // matrices: (keys +0..7, d dn), (keys +8..15, d dn), (keys +0..7, d dn+1), (keys +8..15, d dn+1)
                const int key = kk * 16 + (mi & 1) * 8 + mr;
                const int chunk = dn + (mi >> 1);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vt + key * RB + chunk * 16, b0, b1, b2, b3);
                mma_bf16(o[dn], pf, b0, b1);
                mma_bf16(o[dn + 1], pf, b2, b3);
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);

    // ---- merge the warps ----
    __syncthreads();                                 // every warp is done with its tiles
    float* sm_o = (float*)smem;                      // [WARPS][16][D]
    float* sm_ml = sm_o + WARPS * 16 * D;            // [WARPS][16][2]
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int dn = 0; dn < DN; ++dn) {
            float* p0 = sm_o + ((warp * 16 + r0) * D) + dn * 8 + c0;
            float* p1 = sm_o + ((warp * 16 + r0 + 8) * D) + dn * 8 + c0;
            p0[0] = o[dn][0]; p0[1] = o[dn][1];
            p1[0] = o[dn][2]; p1[1] = o[dn][3];
        }
        if ((lane & 3) == 0) {
            sm_ml[(warp * 16 + r0) * 2] = m[0];      sm_ml[(warp * 16 + r0) * 2 + 1] = l[0];
            sm_ml[(warp * 16 + r0 + 8) * 2] = m[1];  sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = l[1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_rep * D; idx += WARPS * 32) {
        const int r = idx / D, c = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        const float mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = exp2f(sm_ml[(w * 16 + r) * 2] - mb);
            L += f * sm_ml[(w * 16 + r) * 2 + 1];
            O += f * sm_o[(w * 16 + r) * D + c];
        }
        const int h = g * n_rep + r;
        if (n_splits == 1) {
            out[((long long)t * nq + h) * D + c] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else {
            const long long pi = ((long long)e * nq + h) * n_splits + split;
            part_o[pi * D + c] = O;
            if (c == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------
// Head size 128, tiles by TMA.  The pools are seen as matrices [rows, 128] of
// bf16, a row per (page, kv head, token of the page); a tile of 32 keys of one
// kv head is 32 consecutive rows inside one page.  In shared memory a tile is
// two blocks of [32 rows][128 bytes] (elements 0..63 and 64..127) with the
// 128-byte swizzle, so the ldmatrix reads are free of bank conflicts without
// padding.  Differences to the kernel above, beside the copies: scores are
// masked only in the tiles that touch the ends of the key range (whose rows
// outside the range are cleared in shared memory instead of being zero-filled
// by the copy), the running maximum is kept unscaled, and the output is
// rescaled only when some row's maximum has grown.
constexpr int D128 = 128;
constexpr int HALF_TILE_BYTES = TILE * 128;          // one 64-element half of a tile
constexpr int TILE128_BYTES = 2 * HALF_TILE_BYTES;   // K or V tile
constexpr uint32_t TMA_WAIT_LIMIT = 1u << 22;

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
__device__ __forceinline__ void tma_tile_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x,
                                            int row) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(row)
        : "memory");
}
// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a swizzled tile.
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * HALF_TILE_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// CLUSTER: the CTAs of the slices of one (request, kv head) form a thread-block cluster (at most
// 8 slices) and merge their results themselves through distributed shared memory: every CTA
// leaves (max, sum, unnormalised output) of its slice in its own shared memory, and after a
// cluster barrier each CTA works out its share of the output columns from all slices, in slice
// order.  No scratch memory, no second kernel (a kernel of its own costs its place in the chain
// of dependent launches, about 3 us per layer here, whatever little it does).
template <bool FUSED, bool CLUSTER, bool GENERAL>
__global__ void __launch_bounds__(WARPS * 32)
paged_decode_attn_tma_kernel(const __grid_constant__ CUtensorMap k_map,
                             const __grid_constant__ CUtensorMap v_map,
                             const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                             float* __restrict__ part_o, float* __restrict__ part_ml,
                             const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                             const int* __restrict__ block_table, int max_blocks, int num_pages,
                             int page_size, int nq, int nkv, int window, float scale_log2, int n_splits,
                             int* err, const FusedArgs fa) {
    constexpr int D = D128;
    constexpr int KS = D / 16, DN = D / 8;
    constexpr int STAGE_BYTES = 2 * TILE128_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __nv_bfloat16* q_s = (__nv_bfloat16*)(smem + WARPS * NSTAGE * STAGE_BYTES);           // [16][D]
    __nv_bfloat16* row_s = q_s + 16 * D;                                                  // [WARPS][2][D]
    uint64_t* full = (uint64_t*)(row_s + WARPS * 2 * D);                                  // [WARPS][NSTAGE]

    pdl_launch_dependents();
    const bool early = FUSED && fa.has_kv != 0;
    if (!early) pdl_wait();
    const int split = blockIdx.x, g = blockIdx.y, e = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_rep = nq / nkv;
    const int t = cu_q[e];
    // an entry with a prompt portion (or a padding entry without rows) is another kernel's: all
    // CTAs of the entry, which are all CTAs of its cluster, leave here
    if (cu_q[e + 1] - t != 1) return;
    const int pos = kv_len[e] - 1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (long long)e * max_blocks;

    const int first_tile = lo / TILE;
    const int n_tiles = pos / TILE - first_tile + 1;
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int tile_begin = first_tile + split * per_split;
    const int tile_end = min(first_tile + n_tiles, tile_begin + per_split);
    const int n_my = max(0, (tile_end - tile_begin - warp + WARPS - 1) / WARPS);   // this warp's tiles

    const bool makes_kv = FUSED && fa.has_kv != 0;
    const int hi = makes_kv ? pos - 1 : pos;       // last key that is read from the pages

    if (threadIdx.x == 0) {
        for (int i = 0; i < WARPS * NSTAGE; ++i) mbar_init(smem_u32(&full[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const uint32_t wbase = smem_u32(smem) + warp * NSTAGE * STAGE_BYTES;
    const uint32_t wbar = smem_u32(&full[warp * NSTAGE]);
    bool bad_page = false;
    // A tile of 32 keys lies in one page, or, with pages of 8 or 16 tokens, in several: it comes in
    // pieces of `piece` keys (the tensor maps' box), each asked for by a lane of its own.
    const int piece = page_size < TILE ? page_size : TILE;
    const int n_pieces = TILE / piece;
    // lanes 0 .. n_pieces - 1 ask for local tile `idx` (global tile `tile`) of this warp
    auto issue = [&](int idx, int tile) {
        if (lane < n_pieces) {
            // a piece wholly behind the last key or wholly before the window's first one has no page
            // of its own any more (or not yet): the nearest piece that has one is read in its place;
            // its keys are masked by their positions, only the byte count has to be complete
            int key0 = tile * TILE + lane * piece;
            if (key0 > pos) key0 = pos / piece * piece;
            if (key0 + piece <= lo) key0 = lo / piece * piece;
            int page = table[key0 / page_size];
            if (page < 0 || page >= num_pages) {
                bad_page = true;                   // reported below; the copy reads page 0 instead
                page = 0;
            }
            const int row = (page * nkv + g) * page_size + key0 % page_size;
            const uint32_t st = wbase + (idx % NSTAGE) * STAGE_BYTES + lane * piece * 128;
            const uint32_t bar = wbar + (idx % NSTAGE) * 8;
            // the warp's reads of this stage (generic proxy) come before the copies (async proxy)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // (the barrier's phase cannot end before lane 0 has arrived with the byte count, so the
            // other lanes' copies may well land first)
            if (lane == 0) mbar_expect_tx(bar, STAGE_BYTES);
            tma_tile_2d(st, &k_map, bar, 0, row);
            tma_tile_2d(st + HALF_TILE_BYTES, &k_map, bar, 64, row);
            tma_tile_2d(st + TILE128_BYTES, &v_map, bar, 0, row);
            tma_tile_2d(st + TILE128_BYTES + HALF_TILE_BYTES, &v_map, bar, 64, row);
        }
    };
#pragma unroll
    for (int s = 0; s < NSTAGE - 1; ++s)
        if (s < n_my) issue(s, tile_begin + warp + s * WARPS);
    if (early) pdl_wait();                         // from here on q, k and v of this step are read

    // ---- query rows: row r of the MMA tile is query head g * n_rep + r ----
    uint32_t qf[KS][4];
    bool rotate = FUSED && fa.rotary != 0;
    if (FUSED) {
        if (rotate && (pos < 0 || pos >= fa.table_len)) {
            if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_POSITION_RANGE);
            rotate = false;
        }
        if (GENERAL) {
            // another pairing, a partly rotated head, the norm first or (1 + w) weights: row by row
            const long long row_src = (long long)t * fa.qkv_stride;
            for (int i = threadIdx.x; i < 16 * D / 2; i += WARPS * 32) ((uint32_t*)q_s)[i] = 0u;
            __syncthreads();
            for (int r = warp; r < n_rep; r += WARPS)
                rope_norm_row<D, true>(fa, row_src + (long long)(g * n_rep + r) * D, pos, rotate, fa.q_norm_w, lane,
                                       q_s + r * D, nullptr);
            if (makes_kv && pos / TILE >= tile_begin && pos / TILE < tile_end &&
                (pos / TILE - tile_begin) % WARPS == warp) {
                const int page = table[pos / page_size];
                if (page < 0 || page >= num_pages) {
                    bad_page = true;
                } else {
                    const long long prow = (((long long)page * nkv + g) * page_size + pos % page_size) * D;
                    __nv_bfloat16* kv_lin = row_s + warp * 2 * D;              // [key row | value row]
                    rope_norm_row<D, true>(fa, row_src + (long long)(nq + g) * D, pos, rotate, fa.k_norm_w, lane, kv_lin,
                                           fa.k_pool_w + prow);
                    for (int c = 2 * lane; c < D; c += 64) {
                        const float2 x = raw2(fa, row_src + (long long)(nq + nkv + g) * D + c);
                        const __nv_bfloat162 b = __floats2bfloat162_rn(x.x, x.y);
                        *(__nv_bfloat162*)(kv_lin + D + c) = b;
                        *(__nv_bfloat162*)(fa.v_pool_w + prow + c) = b;
                    }
                }
            }
        } else {
            // this lane's cosines, sines and norm weights are the same for every query row; the
            // loads of two rows and of the tables are in flight together
            static_assert(RowRegs<D>::IT == 1, "head size 128: one pair of neighbours per lane and half");
            float2 cs[1], sn[1], w1[1], w2[1];
            const int j = 2 * lane;
            const bool norm = fa.q_norm_w != nullptr;
            cs[0] = sn[0] = w1[0] = w2[0] = make_float2(0.f, 0.f);
            if (rotate) {
                cs[0] = *(const float2*)(fa.cos_tab + (long long)pos * (D / 2) + j);
                sn[0] = *(const float2*)(fa.sin_tab + (long long)pos * (D / 2) + j);
            }
            if (norm) {
                w1[0] = *(const float2*)(fa.q_norm_w + j);
                w2[0] = *(const float2*)(fa.q_norm_w + j + D / 2);
            }
            const long long row_src = (long long)t * fa.qkv_stride;
            const long long q_src = row_src + (long long)(g * n_rep) * D;
            auto load_two = [&](int r, RowRegs<D>& ra, RowRegs<D>& rb) {
                // rows r and r + WARPS of the group: four places, one round of loads
                const bool two = r + WARPS < n_rep;
                const long long at[4] = {q_src + (long long)r * D + j, q_src + (long long)r * D + j + D / 2,
                                         q_src + (long long)(r + WARPS) * D + j,
                                         q_src + (long long)(r + WARPS) * D + j + D / 2};
                float2 got[4];
                raw2x4(fa, at, two ? 4 : 2, got);
                ra.u[0] = got[0]; ra.v[0] = got[1];
                rb.u[0] = got[2]; rb.v[0] = got[3];
            };
            RowRegs<D> ra, rb;
            if (warp < n_rep) load_two(warp, ra, rb);
            for (int i = threadIdx.x; i < 16 * D / 2; i += WARPS * 32) ((uint32_t*)q_s)[i] = 0u;
            __syncthreads();
            for (int r = warp; r < n_rep; r += 2 * WARPS) {
                if (r != warp) load_two(r, ra, rb);
                row_finish<D>(ra, rotate, cs, sn, norm, w1, w2, fa.eps, lane, q_s + r * D, nullptr);
                if (r + WARPS < n_rep)
                    row_finish<D>(rb, rotate, cs, sn, norm, w1, w2, fa.eps, lane, q_s + (r + WARPS) * D, nullptr);
            }
            // The warp whose tiles include the new position makes that position's key (encoded,
            // normalised) and value now, for the page and, kept in shared memory, for its tile later:
            // at the end of the loop these loads and the arithmetic would lengthen the whole kernel.
            if (makes_kv && pos / TILE >= tile_begin && pos / TILE < tile_end &&
                (pos / TILE - tile_begin) % WARPS == warp) {
                const int page = table[pos / page_size];
                if (page < 0 || page >= num_pages) {
                    bad_page = true;
                } else {
                    const long long prow = (((long long)page * nkv + g) * page_size + pos % page_size) * D;
                    const long long k_src = row_src + (long long)(nq + g) * D, v_src = row_src + (long long)(nq + nkv + g) * D;
                    const long long at[4] = {k_src + j, k_src + j + D / 2, v_src + j, v_src + j + D / 2};
                    float2 got[4];
                    raw2x4(fa, at, 4, got);
                    RowRegs<D> rk;
                    rk.u[0] = got[0]; rk.v[0] = got[1];
                    float2 kw1[1], kw2[1];
                    kw1[0] = kw2[0] = make_float2(0.f, 0.f);
                    const bool knorm = fa.k_norm_w != nullptr;
                    if (knorm) {
                        kw1[0] = *(const float2*)(fa.k_norm_w + j);
                        kw2[0] = *(const float2*)(fa.k_norm_w + j + D / 2);
                    }
                    __nv_bfloat16* kv_lin = row_s + warp * 2 * D;              // [key row | value row]
                    row_finish<D>(rk, rotate, cs, sn, knorm, kw1, kw2, fa.eps, lane, kv_lin, fa.k_pool_w + prow);
                    const __nv_bfloat162 va = __floats2bfloat162_rn(got[2].x, got[2].y);
                    const __nv_bfloat162 vb = __floats2bfloat162_rn(got[3].x, got[3].y);
                    *(__nv_bfloat162*)(kv_lin + D + j) = va;
                    *(__nv_bfloat162*)(kv_lin + D + j + D / 2) = vb;
                    *(__nv_bfloat162*)(fa.v_pool_w + prow + j) = va;
                    *(__nv_bfloat162*)(fa.v_pool_w + prow + j + D / 2) = vb;
                }
            }
        }
        __syncthreads();
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                qf[ks][i] = *(const uint32_t*)(q_s + (r0 + (i & 1) * 8) * D + ks * 16 + c0 + (i >> 1) * 8);
    } else {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = r0 + (i & 1) * 8, c = ks * 16 + c0 + (i >> 1) * 8;
                uint32_t v = 0;
                if (r < n_rep)
                    v = *(const uint32_t*)(q + ((long long)t * nq + g * n_rep + r) * D + c);
                qf[ks][i] = v;
            }
        }
    }

    float o[DN][4];
#pragma unroll
    for (int i = 0; i < DN; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};     // m: unscaled maximum of the raw scores

    // per-lane parts of the ldmatrix addresses
    const int mi = lane >> 3, mr = lane & 7;
    const uint32_t k_lane = (uint32_t)(((mi >> 1) * 8 + mr) * 128);   // + half * 16 rows
    const uint32_t k_x = (uint32_t)(((mi & 1) ^ mr) << 4);            // chunk = ks * 2 + (mi & 1)
    const uint32_t v_lane = (uint32_t)(((mi & 1) * 8 + mr) * 128);    // + kk * 16 rows
    const uint32_t v_x = (uint32_t)(((mi >> 1) ^ mr) << 4);           // chunk = dn + (mi >> 1)
    bool timed_out = false;

    for (int it = 0; it < n_my; ++it) {
        const int ti = tile_begin + warp + it * WARPS;
        if (it + NSTAGE - 1 < n_my) issue(it + NSTAGE - 1, ti + (NSTAGE - 1) * WARPS);
        const uint32_t kt = wbase + (it % NSTAGE) * STAGE_BYTES, vt = kt + TILE128_BYTES;
        {
            const uint32_t bar = wbar + (it % NSTAGE) * 8, parity = (it / NSTAGE) & 1;
            uint32_t spin = 0;
            while (!mbar_try_wait(bar, parity))
                if (++spin > TMA_WAIT_LIMIT) { timed_out = true; break; }
            if (timed_out) break;
        }
        const bool edge = ti * TILE < lo || ti * TILE + TILE - 1 > hi;
        if (edge) {
            // rows outside [lo, hi] hold whatever the page holds: clear them (the scores of such
            // keys are masked below, a cleared value row keeps 0 * garbage out of the output)
            uint8_t* stage = smem + (size_t)(warp * NSTAGE + it % NSTAGE) * STAGE_BYTES;
            for (int r = lane >> 4; r < TILE; r += 2) {
                const int j = ti * TILE + r;
                if (j < lo || j > hi) {
                    const int c = lane & 15;
                    *(uint4*)(stage + sw_off(r, c)) = make_uint4(0u, 0u, 0u, 0u);
                    *(uint4*)(stage + TILE128_BYTES + sw_off(r, c)) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            __syncwarp();
            if (makes_kv && ti == pos / TILE) {
                // this tile holds the new position: its key and value, made before the loop, go
                // into the tile in shared memory
                const __nv_bfloat16* kv_lin = row_s + warp * 2 * D;
                const int r = pos % TILE;
                if (lane < 16) *(uint4*)(stage + sw_off(r, lane)) = *(const uint4*)(kv_lin + lane * 8);
                else *(uint4*)(stage + TILE128_BYTES + sw_off(r, lane - 16)) = *(const uint4*)(kv_lin + D + (lane - 16) * 8);
                __syncwarp();
            }
        }

        // ---- scores: 16 rows x 32 keys ----
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                // matrices: (keys +0..7, d lo), (keys +0..7, d hi), (keys +8..15, d lo), (keys +8..15, d hi)
                const uint32_t addr = kt + (ks >> 2) * HALF_TILE_BYTES + half * 16 * 128 + k_lane +
                                      ((uint32_t)(((ks & 3) * 2) << 4) ^ k_x);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(addr, b0, b1, b2, b3);
                mma_bf16(s[half * 2], qf[ks], b0, b1);
                mma_bf16(s[half * 2 + 1], qf[ks], b2, b3);
            }
        }
        // ---- running softmax ----
        if (edge) {
            const int key0 = ti * TILE + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = key0 + nt * 8 + (c & 1);
                    if (j < lo || j > pos) s[nt][c] = -INFINITY;
                }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) mx[c >> 1] = fmaxf(mx[c >> 1], s[nt][c]);
        float m_new[2], base[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_new[h] = fmaxf(m[h], quad_max(mx[h]));
            base[h] = (m_new[h] == -INFINITY) ? 0.f : m_new[h] * scale_log2;
        }
        if (__any_sync(0xffffffffu, m_new[0] != m[0] || m_new[1] != m[1])) {
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                corr[h] = exp2f(m[h] * scale_log2 - base[h]);       // exp2(-inf) = 0 on the first tile
                m[h] = m_new[h];
                l[h] *= corr[h];
            }
#pragma unroll
            for (int i = 0; i < DN; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = exp2f(fmaf(s[nt][c], scale_log2, -base[c >> 1]));
                s[nt][c] = p;
                rs[c >> 1] += p;
            }
        l[0] += rs[0];
        l[1] += rs[1];
        // ---- output += p v ----
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dn = 0; dn < DN; dn += 2) {
                // matrices: (keys +0..7, d dn), (keys +8..15, d dn), (keys +0..7, d dn+1), (keys +8..15, d dn+1)
                const uint32_t addr = vt + (dn >> 3) * HALF_TILE_BYTES + kk * 16 * 128 + v_lane +
                                      ((uint32_t)((dn & 7) << 4) ^ v_x);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(addr, b0, b1, b2, b3);
                mma_bf16(o[dn], pf, b0, b1);
                mma_bf16(o[dn + 1], pf, b2, b3);
            }
        }
        __syncwarp();
    }
    if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    if (__any_sync(0xffffffffu, timed_out)) {
        if (lane == 0) atomicOr(err, CRANE_ERR_WAIT_TIMEOUT);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);     // copies may still be landing
    }
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);
    // from here on the maximum counts in the units of the scaled scores
    m[0] *= scale_log2;
    m[1] *= scale_log2;

    // ---- merge the warps ----
    __syncthreads();                                 // every warp is done with its tiles
    float* sm_o = (float*)smem;                      // [WARPS][16][D]
    float* sm_ml = sm_o + WARPS * 16 * D;            // [WARPS][16][2]
    float* cl_ml = sm_ml + WARPS * 16 * 2;           // [16][2]  this slice's (max, sum), for the cluster's merge
    float* cl_o = cl_ml + 16 * 2;                    // [16][D]  and its unnormalised output
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int dn = 0; dn < DN; ++dn) {
            float* p0 = sm_o + ((warp * 16 + r0) * D) + dn * 8 + c0;
            float* p1 = sm_o + ((warp * 16 + r0 + 8) * D) + dn * 8 + c0;
            p0[0] = o[dn][0]; p0[1] = o[dn][1];
            p1[0] = o[dn][2]; p1[1] = o[dn][3];
        }
        if ((lane & 3) == 0) {
            sm_ml[(warp * 16 + r0) * 2] = m[0];      sm_ml[(warp * 16 + r0) * 2 + 1] = l[0];
            sm_ml[(warp * 16 + r0 + 8) * 2] = m[1];  sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = l[1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_rep * D; idx += WARPS * 32) {
        const int r = idx / D, c = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        const float mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = exp2f(sm_ml[(w * 16 + r) * 2] - mb);
            L += f * sm_ml[(w * 16 + r) * 2 + 1];
            O += f * sm_o[(w * 16 + r) * D + c];
        }
        const int h = g * n_rep + r;
        if (n_splits == 1) {
            out[((long long)t * nq + h) * D + c] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else if (CLUSTER) {
            cl_o[r * D + c] = O;
            if (c == 0) { cl_ml[r * 2] = M; cl_ml[r * 2 + 1] = L; }
        } else {
            const long long pi = ((long long)e * nq + h) * n_splits + split;
            part_o[pi * D + c] = O;
            if (c == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
    if (CLUSTER && n_splits > 1) {
        // every slice's result is in its CTA's shared memory; this CTA takes its share of the
        // n_rep x D outputs and reads that element of every slice (slice s = cluster rank s)
        asm volatile("barrier.cluster.arrive.release.aligned;\n"
                     "barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int total = n_rep * D;
        const int begin = (int)((long long)split * total / n_splits), end = (int)((long long)(split + 1) * total / n_splits);
        const uint32_t o_addr = smem_u32(cl_o), ml_addr = smem_u32(cl_ml);
        for (int idx = begin + (int)threadIdx.x; idx < end; idx += WARPS * 32) {
            const int r = idx / D;
            float2 ml[8];
            float ov[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                ml[sp] = make_float2(-INFINITY, 0.f);
                ov[sp] = 0.f;
                if (sp < n_splits) {
                    uint32_t ra, rb;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(ml_addr + (uint32_t)(r * 8)), "r"(sp));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(o_addr + (uint32_t)(idx * 4)), "r"(sp));
                    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(ml[sp].x), "=f"(ml[sp].y) : "r"(ra) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ov[sp]) : "r"(rb) : "memory");
                }
            }
            float M = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) M = fmaxf(M, ml[sp].x);
            const float mb = (M == -INFINITY) ? 0.f : M;
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                const float f = exp2f(ml[sp].x - mb);        // 0 beyond n_splits
                L += f * ml[sp].y;
                acc += f * ov[sp];
            }
            out[((long long)t * nq + g * n_rep + r) * D + (idx % D)] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        }
        // nobody leaves while a CTA of the cluster may still read its shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;\n"
                     "barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
}

// One thread per output column: the (max, sum) pairs and this column of up to MAXS slices,
// all loads in flight together, added in slice order.
template <int MAXS>
__device__ __forceinline__ void merge_column(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                             __nv_bfloat16* __restrict__ out, long long base, int t, int nq,
                                             int h, int d, int n_splits) {
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float2 ml[MAXS];
        float o[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
            ml[s] = s < n_splits ? *(const float2*)(part_ml + (base + s) * 2) : make_float2(-INFINITY, 0.f);
            o[s] = s < n_splits ? part_o[(base + s) * d + c] : 0.f;
        }
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < MAXS; ++s) M = fmaxf(M, ml[s].x);
        const float mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
            const float f = exp2f(ml[s].x - mb);           // 0 for the slices beyond n_splits
            L += f * ml[s].y;
            acc += f * o[s];
        }
        out[((long long)t * nq + h) * d + c] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
}

// out[t, h, :] = sum_s w_s o_s / sum_s w_s l_s with w_s = exp2(m_s - max m).
// One CTA per (request, query head), a thread per output column.  Up to 32 slices: every
// thread fetches the slices' (max, sum) pairs and its column of their outputs with all loads
// in flight together and works the weights out itself.  More slices: the pairs are fetched by
// one thread each, the weights go through shared memory, and the outputs are summed with
// four loads in flight per thread.  Always in slice order.
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q,
                                    int nq, int d, int n_splits) {
    __shared__ float wgt[64];
    __shared__ float m_s[64], l_s[64];
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, h = blockIdx.y;
    const long long base = ((long long)e * nq + h) * n_splits;
    const int t = cu_q[e];
    if (cu_q[e + 1] - t != 1) return;
    if (n_splits <= 64) {
        // all loads of a thread go out together; 16 slices' worth of registers when that is enough
        if (n_splits <= 16) merge_column<16>(part_o, part_ml, out, base, t, nq, h, d, n_splits);
        else if (n_splits <= 32) merge_column<32>(part_o, part_ml, out, base, t, nq, h, d, n_splits);
        else merge_column<64>(part_o, part_ml, out, base, t, nq, h, d, n_splits);
        return;
    }
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
        m_s[s] = part_ml[(base + s) * 2];
        l_s[s] = part_ml[(base + s) * 2 + 1];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float M = -INFINITY;
        for (int s = 0; s < n_splits; ++s) M = fmaxf(M, m_s[s]);
        const float mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float f = exp2f(m_s[s] - mb);
            L += f * l_s[s];
            wgt[s] = f;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int s = 0; s < n_splits; ++s) wgt[s] *= inv;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float* po = part_o + base * d + c;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        int s = 0;
        for (; s + 4 <= n_splits; s += 4) {
            const float v0 = po[(long long)s * d], v1 = po[(long long)(s + 1) * d];
            const float v2 = po[(long long)(s + 2) * d], v3 = po[(long long)(s + 3) * d];
            a0 += wgt[s] * v0;
            a1 += wgt[s + 1] * v1;
            a2 += wgt[s + 2] * v2;
            a3 += wgt[s + 3] * v3;
        }
        for (; s < n_splits; ++s) a0 += wgt[s] * po[(long long)s * d];
        out[((long long)t * nq + h) * d + c] = __float2bfloat16_rn((a0 + a1) + (a2 + a3));
    }
}

// ---- host side of the TMA path ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (EncodeTiledFn)sym;
    }
    return fn;
}
// CRANE_DECODE_TMA=0 keeps the cp.async kernel at head size 128 too.
bool tma_path_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("CRANE_DECODE_TMA");
        on = (v == nullptr || v[0] != '0') ? 1 : 0;
    }
    return on == 1;
}
// CRANE_DECODE_CLUSTER=0: the slices always go through scratch memory and the merge kernel.
bool cluster_merge_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("CRANE_DECODE_CLUSTER");
        on = (v == nullptr || v[0] != '0') ? 1 : 0;
    }
    return on == 1;
}
// The pool as [rows, 128] bf16; box of 64 elements x box_rows rows (a tile's 32, or a page's 8 or 16),
// 128-byte swizzle.
bool pool_map(CUtensorMap* map, const void* pool, long long rows, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || ((uintptr_t)pool & 15)) return false;
    cuuint64_t dims[2] = {(cuuint64_t)D128, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D128 * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool FUSED, bool GENERAL>
int launch_decode_tma(const void* q, void* out, float* part_o, float* part_ml, const void* k_pool,
                      const void* v_pool, const int* cu_q, const int* kv_len, const int* block_table,
                      int max_blocks, int num_pages, int page_size, int nq, int nkv, int window,
                      float scale, int n_splits, int* err, const FusedArgs& fa, dim3 grid, bool cluster,
                      cudaStream_t st) {
    constexpr int tiles = WARPS * NSTAGE * 2 * TILE128_BYTES + 16 * D128 * 2 + WARPS * 2 * D128 * 2 +
                          WARPS * NSTAGE * 8;
    constexpr int merge = (WARPS + 1) * 16 * (D128 + 2) * 4;
    constexpr int smem = (tiles > merge ? tiles : merge) + 1024;
    CUtensorMap km, vm;
    const long long rows = (long long)num_pages * nkv * page_size;
    const int box_rows = page_size < TILE ? page_size : TILE;
    if (!pool_map(&km, k_pool, rows, box_rows) || !pool_map(&vm, v_pool, rows, box_rows))
        return (int)cudaErrorInvalidValue;
    if (cluster) {
        auto kern = paged_decode_attn_tma_kernel<FUSED, true, GENERAL>;
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                return (int)cudaGetLastError();
            configured = true;
        }
        return crane_launch_cluster(kern, grid, dim3(WARPS * 32), smem, dim3(grid.x, 1, 1), st, km, vm,
                                    (const __nv_bfloat16*)q, (__nv_bfloat16*)out, part_o, part_ml, cu_q, kv_len,
                                    block_table, max_blocks, num_pages, page_size, nq, nkv, window,
                                    scale * 1.4426950408889634f, n_splits, err, fa);
    }
    auto kern = paged_decode_attn_tma_kernel<FUSED, false, GENERAL>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return crane_launch(kern, grid, dim3(WARPS * 32), smem, st, km, vm, (const __nv_bfloat16*)q,
                        (__nv_bfloat16*)out, part_o, part_ml, cu_q, kv_len, block_table, max_blocks,
                        num_pages, page_size, nq, nkv, window, scale * 1.4426950408889634f, n_splits, err,
                        fa);
}

template <int D, bool FUSED, bool GENERAL>
int launch_decode(const void* q, void* out, float* part_o, float* part_ml, const void* k_pool,
                  const void* v_pool, const int* cu_q, const int* kv_len, const int* block_table,
                  int max_blocks, int num_pages, int page_size, int n_entries, int nq, int nkv,
                  int window, float scale, int n_splits, int* err, const FusedArgs& fa, cudaStream_t st) {
    constexpr int tiles = WARPS * NSTAGE * 2 * TILE * Tile<D>::ROW_BYTES + (FUSED ? 16 * D * 2 : 0);
    constexpr int merge = WARPS * 16 * (D + 2) * 4;
    constexpr int smem = tiles > merge ? tiles : merge;
    auto kern = paged_decode_attn_kernel<D, FUSED, GENERAL>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    dim3 grid(n_splits, nkv, n_entries);
    // pages of whole tiles, or tiles of whole pages (8 or 16 tokens: a piece of a tile is then a multiple
    // of the 1024 bytes the swizzle pattern repeats after)
    const bool pages_fit = page_size % TILE == 0 || (page_size >= 8 && TILE % page_size == 0);
    if (D == D128 && pages_fit && tma_path_enabled()) {
        // 2 to 8 slices merge themselves in a cluster; more go through scratch memory and a second kernel
        const bool cluster = n_splits > 1 && n_splits <= 8 && cluster_merge_enabled();
        const int rc = launch_decode_tma<FUSED, GENERAL>(q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len,
                                                block_table, max_blocks, num_pages, page_size, nq, nkv,
                                                window, scale, n_splits, err, fa, grid, cluster, st);
        if (rc != 0) return rc;
        if (n_splits > 1 && !cluster)
            return crane_launch(decode_merge_kernel, dim3(n_entries, nq), dim3(D >= 128 ? 128 : 64), 0, st,
                                (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, cu_q, nq,
                                D, n_splits);
        return 0;
    }
    int rc = crane_launch(kern, grid, dim3(WARPS * 32), smem, st, (const __nv_bfloat16*)q,
                          (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)k_pool,
                          (const __nv_bfloat16*)v_pool, cu_q, kv_len, block_table, max_blocks, num_pages,
                          page_size, nq, nkv, window, scale * 1.4426950408889634f, n_splits, err, fa);
    if (rc == 0 && n_splits > 1)
        rc = crane_launch(decode_merge_kernel, dim3(n_entries, nq), dim3(D >= 128 ? 128 : 64), 0, st,
                          (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, cu_q, nq, D,
                          n_splits);
    return rc;
}
}  // namespace

// Every head size is compiled as an object of its own from this file (the build passes
// CRANE_HEAD_SIZE), in parallel: such an object holds nothing but that size's kernels and the
// launcher below.  The object without CRANE_HEAD_SIZE holds the entry points, which pick a launcher.
#define CRANE_CAT2(a, b) a##b
#define CRANE_CAT(a, b) CRANE_CAT2(a, b)
#define CRANE_DECODE_LAUNCHER_ARGS                                                                   \
    int fused, const void *q, void *out, float *part_o, float *part_ml, const void *k_pool,           \
        const void *v_pool, const int *cu_q, const int *kv_len, const int *block_table, int max_blocks, \
        int num_pages, int page_size, int n_entries, int nq, int nkv, int window, float scale,         \
        int n_splits, int *err, const void *fused_args, cudaStream_t st
#ifdef CRANE_HEAD_SIZE
extern "C" int CRANE_CAT(crane_decode_launch_d, CRANE_HEAD_SIZE)(CRANE_DECODE_LAUNCHER_ARGS) {
    const FusedArgs& fa = *(const FusedArgs*)fused_args;
#define CRANE_DECODE_CALL(F, G)                                                                        \
    launch_decode<CRANE_HEAD_SIZE, F, G>(q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, block_table, \
                                         max_blocks, num_pages, page_size, n_entries, nq, nkv, window, scale, \
                                         n_splits, err, fa, st)
    if (fused) return fa.general ? CRANE_DECODE_CALL(true, true) : CRANE_DECODE_CALL(true, false);
    return CRANE_DECODE_CALL(false, false);
#undef CRANE_DECODE_CALL
}
#else
// The head sizes whose objects are linked into this library: all that there are, or the ones the build
// names (-D"CRANE_HEAD_SIZE_LIST(X)=X(64) X(128)": a library for the models at hand compiles faster).
#ifdef CRANE_HEAD_SIZE_LIST
#define CRANE_DECODE_HEAD_SIZES(X) CRANE_HEAD_SIZE_LIST(X)
#else
#define CRANE_DECODE_HEAD_SIZES(X) X(16) X(32) X(48) X(64) X(80) X(96) X(112) X(128) X(160) X(192) X(256)
#endif
#define DECLARE(DD) extern "C" int crane_decode_launch_d##DD(CRANE_DECODE_LAUNCHER_ARGS);
CRANE_DECODE_HEAD_SIZES(DECLARE)
#undef DECLARE

namespace {
int launch_for_head_size(int d, CRANE_DECODE_LAUNCHER_ARGS) {
#define CASE(DD)                                                                                     \
    case DD:                                                                                         \
        return crane_decode_launch_d##DD(fused, q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, \
                                         block_table, max_blocks, num_pages, page_size, n_entries, nq, \
                                         nkv, window, scale, n_splits, err, fused_args, st);
    switch (d) { CRANE_DECODE_HEAD_SIZES(CASE) }
#undef CASE
    return (int)cudaErrorInvalidValue;
}
}  // namespace

// 1 if the kernel is built for this head size and group size, else 0.
CRANE_API int crane_paged_decode_attention_supports(int d, int nq, int nkv) {
    if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16) return 0;
#define IS(DD) if (d == DD) return 1;
    CRANE_DECODE_HEAD_SIZES(IS)
#undef IS
    return 0;
}

// The entries with exactly one token (row cu_q[e] of q and out); entries with
// more or no rows are skipped, so that a step's prompt portions can go to the
// prefill kernel and its decoded tokens here.  part_o needs
// n_entries * nq * n_splits * d floats and part_ml n_entries * nq * n_splits * 2
// when n_splits > 1.
CRANE_API int crane_paged_decode_attention(const void* q, void* out, float* part_o, float* part_ml,
                                           const void* k_pool, const void* v_pool, const int* cu_q,
                                           const int* kv_len, const int* block_table, int max_blocks,
                                           int num_pages, int page_size, int n_entries, int nq, int nkv,
                                           int d, int window, float scale, int n_splits, int* err,
                                           cudaStream_t st) {
    if (n_entries <= 0) return 0;
    if (!crane_paged_decode_attention_supports(d, nq, nkv) || n_splits < 1 || n_splits > 64)
        return (int)cudaErrorInvalidValue;
    const FusedArgs none = {};
    return launch_for_head_size(d, 0, q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, block_table,
                                max_blocks, num_pages, page_size, n_entries, nq, nkv, window, scale,
                                n_splits, err, &none, st);
}

// The fused form: q, k and v of the step's tokens come raw from the product
// (`qkv` whole, or `qkv_parts` as n_parts float partial sums), one row of
// [q | k | v] (q alone when has_kv == 0) per token.  The kernel encodes and
// normalises them, writes the new key and value into their pages and attends; a
// second kernel merges the slices.  Head sizes must be multiples of 4.
CRANE_API int crane_paged_decode_attention_fused(
    const void* qkv, const float* qkv_parts, int n_parts, long long part_stride, int qkv_stride,
    int has_kv, int rotary, const float* cos_tab, const float* sin_tab, int table_len,
    const float* q_norm_w, const float* k_norm_w, float eps, void* out, float* part_o, float* part_ml,
    void* k_pool, void* v_pool, const int* cu_q, const int* kv_len,
    const int* block_table, int max_blocks, int num_pages, int page_size, int n_entries, int nq, int nkv,
    int d, int window, float scale, int n_splits, int rotary_dim, int interleaved, int norm_first,
    float norm_offset, int* err, cudaStream_t st) {
    if (n_entries <= 0) return 0;
    if (rotary_dim <= 0) rotary_dim = d;
    if (!crane_paged_decode_attention_supports(d, nq, nkv) || n_splits < 1 || n_splits > 64 || (d & 3) ||
        (qkv_stride & 1) || (part_stride & 1) || rotary_dim > d || (rotary_dim & 1))
        return (int)cudaErrorInvalidValue;
    FusedArgs fa;
    fa.rope = RopeParams{rotary_dim, interleaved ? 1 : 0, norm_first ? 1 : 0, norm_offset};
    fa.general = rope_is_default(fa.rope, d) ? 0 : 1;
    fa.qkv = (const __nv_bfloat16*)qkv; fa.qkv_parts = qkv_parts; fa.n_parts = n_parts;
    fa.part_stride = part_stride; fa.qkv_stride = qkv_stride; fa.has_kv = has_kv; fa.rotary = rotary;
    fa.cos_tab = cos_tab; fa.sin_tab = sin_tab; fa.table_len = table_len; fa.q_norm_w = q_norm_w;
    fa.k_norm_w = k_norm_w; fa.eps = eps; fa.k_pool_w = (__nv_bfloat16*)k_pool;
    fa.v_pool_w = (__nv_bfloat16*)v_pool;
    return launch_for_head_size(d, 1, nullptr, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len,
                                block_table, max_blocks, num_pages, page_size, n_entries, nq, nkv, window,
                                scale, n_splits, err, &fa, st);
}

// ------------------------------------------------------------------------
// The entry point that allocates nothing (declared and described in
// no_alloc.h).  The slices' partial results live in this array of the library
// image: first the unnormalised outputs, then the (max, sum) pairs.
static __device__ __align__(256) float g_noalloc_scratch[CRANE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES];      // device address of the array, per device, once looked up

// In host code the array's name is only a handle: the address a kernel can use
// has to be asked for, with the device in question current.
int scratch_address(float** out) {
    int dev = -1;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess) return (int)rc;
    if (dev < 0 || dev >= MAX_DEVICES) return CRANE_NOALLOC_BAD_ARGUMENT;
    if (g_scratch_addr[dev] == nullptr) {
        float* p = nullptr;
        rc = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (rc != cudaSuccess || p == nullptr) return rc != cudaSuccess ? (int)rc : CRANE_NOALLOC_NO_SYMBOL;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}
}  // namespace

CRANE_API const char* crane_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case CRANE_NOALLOC_TOO_LARGE:
            return "n_entries * nq * n_splits * (d + 2) floats exceed the library's built-in scratch "
                   "array (CRANE_NOALLOC_SCRATCH_FLOATS = 1048576 floats): use fewer slices, fewer "
                   "entries per call, or the entry point that takes the caller's scratch buffers";
        case CRANE_NOALLOC_BAD_ARGUMENT:
            return "an argument is out of range (head size or head grouping without a kernel, "
                   "n_splits outside 1..64, or a device ordinal beyond 63)";
        case CRANE_NOALLOC_NO_SYMBOL:
            return "the device address of the built-in scratch array could not be found";
    }
    return "a CUDA error (positive codes are cudaError_t values)";
}

CRANE_API int crane_paged_decode_attention_noalloc(const void* q, void* out, const void* k_pool,
                                                   const void* v_pool, const int* cu_q,
                                                   const int* kv_len, const int* block_table,
                                                   int max_blocks, int num_pages, int page_size,
                                                   int n_entries, int nq, int nkv, int d, int window,
                                                   float scale, int n_splits, int* err,
                                                   cudaStream_t stream) {
    if (n_entries <= 0) return 0;
    if (!crane_paged_decode_attention_supports(d, nq, nkv) || n_splits < 1 || n_splits > 64)
        return CRANE_NOALLOC_BAD_ARGUMENT;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (n_splits > 1) {
        const long long slots = (long long)n_entries * nq * n_splits;
        if (slots * (d + 2) > (long long)CRANE_NOALLOC_SCRATCH_FLOATS) return CRANE_NOALLOC_TOO_LARGE;
        float* base = nullptr;
        const int rc = scratch_address(&base);
        if (rc != 0) return rc;
        part_o = base;                   // [slots][d]
        part_ml = base + slots * d;      // [slots][2]
    }
    return crane_paged_decode_attention(q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len,
                                        block_table, max_blocks, num_pages, page_size, n_entries, nq,
                                        nkv, d, window, scale, n_splits, err, stream);
}
#endif  // CRANE_HEAD_SIZE
