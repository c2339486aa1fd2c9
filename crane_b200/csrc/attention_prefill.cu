// Attention of prompt portions (and whatever else is in the batch) over the
// paged cache in bf16: online-softmax ("flash") attention, one CTA per tile of
// 64 query rows of one request and one query head, four warps of 16 rows each,
// keys and values streamed through shared memory in tiles of 64.  A request's
// rows sit at positions kv_len - q_len .. kv_len - 1 and row i reads the keys
// max(0, p_i - window + 1) .. p_i of its own request through the block table,
// so portions cut anywhere, single decoded tokens and whole prompts are all
// the same case.
//
// scores = q k^T / sqrt(d), causal, softmax in float, query head h reads kv
// head h / (nq / nkv): crane-core/src/models/hunyuan_dense/modeling.rs:611-636,
// 1012-1033.  The reference materialises the [S, T] scores and a host-built
// mask; here neither exists.
#include "attention_mma.cuh"

namespace {
using namespace attn;

constexpr int BQ = 64;      // query rows per CTA
constexpr int BKV = 64;     // keys per tile
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;

template <int D>
__global__ void __launch_bounds__(THREADS, 3)
paged_prefill_attn_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                          const __nv_bfloat16* __restrict__ k_pool,
                          const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ cu_q,
                          const int* __restrict__ kv_len, const int* __restrict__ block_table,
                          int max_blocks, int num_pages, int page_size, int n_entries, int nq, int nkv,
                          int window, float scale_log2, int skip_single, int* err) {
    constexpr int RB = Tile<D>::ROW_BYTES;
    constexpr int TILE_BYTES = BKV * RB;
    constexpr int KS = D / 16, DN = D / 8;
    extern __shared__ __align__(16) uint8_t smem[];

    // which request and which of its query tiles this CTA has; a request's last tiles (which
    // read the most keys) come first, so that the long CTAs start early
    // (CTAs go to the SMs in the order of their index, heads fastest: all heads of a long tile first)
    int e = 0, tile = blockIdx.y;
    for (; e < n_entries; ++e) {
        const int rows = cu_q[e + 1] - cu_q[e];
        // skip_single: entries of one token have no tile here (the decode kernel takes them)
        const int tiles = (skip_single && rows == 1) ? 0 : (rows + BQ - 1) / BQ;
        if (tile < tiles) {
            tile = tiles - 1 - tile;
            break;
        }
        tile -= tiles;
    }
    if (e >= n_entries) return;
    const int h = blockIdx.x, g = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = cu_q[e], q_len = cu_q[e + 1] - row0;
    const int pos0 = kv_len[e] - q_len;                  // position of the request's first row
    const int r_begin = tile * BQ, r_end = min(q_len, r_begin + BQ);
    const int* table = block_table + (long long)e * max_blocks;

    // rows of this thread: ra and ra + 8 within the warp's 16
    const int ra = r_begin + warp * 16 + (lane >> 2), rb = ra + 8;
    const int pa = pos0 + ra, pb = pos0 + rb;            // their positions
    uint32_t qf[KS][4];
    {
        const int c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = (i & 1) ? rb : ra, c = ks * 16 + c0 + (i >> 1) * 8;
                qf[ks][i] = r < r_end ? *(const uint32_t*)(q + ((long long)(row0 + r) * nq + h) * D + c) : 0u;
            }
    }
    float o[DN][4];
#pragma unroll
    for (int i = 0; i < DN; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    bool bad_page = false;

    // keys that any row of the CTA reads
    const int p_first = pos0 + r_begin, p_last = pos0 + r_end - 1;
    const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int t_begin = lo / BKV, t_end = p_last / BKV + 1;
    // this warp's rows span positions wp_first .. wp_last
    const int wp_first = pos0 + r_begin + warp * 16;
    const int wp_last = min(p_last, wp_first + 15);

    const uint32_t sbase = smem_u32(smem);
    load_tile_async<D, BKV, THREADS>(sbase, k_pool, table, num_pages, page_size, nkv, g, t_begin * BKV,
                                     lo, p_last, threadIdx.x, bad_page);
    load_tile_async<D, BKV, THREADS>(sbase + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g,
                                     t_begin * BKV, lo, p_last, threadIdx.x, bad_page);
    cp_async_commit();
    for (int ti = t_begin, it = 0; ti < t_end; ++ti, ++it) {
        const uint32_t kt = sbase + (it & 1) * 2 * TILE_BYTES, vt = kt + TILE_BYTES;
        if (ti + 1 < t_end) {
            const uint32_t nk = sbase + ((it + 1) & 1) * 2 * TILE_BYTES;
            load_tile_async<D, BKV, THREADS>(nk, k_pool, table, num_pages, page_size, nkv, g,
                                             (ti + 1) * BKV, lo, p_last, threadIdx.x, bad_page);
            load_tile_async<D, BKV, THREADS>(nk + TILE_BYTES, v_pool, table, num_pages, page_size, nkv,
                                             g, (ti + 1) * BKV, lo, p_last, threadIdx.x, bad_page);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const int key_base = ti * BKV;
        // a warp skips tiles that lie wholly after its last row or before its first row's window
        const bool skip = key_base > wp_last ||
                          (window > 0 && key_base + BKV - 1 < wp_first - window + 1) ||
                          wp_first > p_last;
        if (!skip) {
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
            const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int key = q4 * 16 + (mi >> 1) * 8 + mr;
                    const int chunk = ks * 2 + (mi & 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(kt + key * RB + chunk * 16, b0, b1, b2, b3);
                    mma_bf16(s[q4 * 2], qf[ks], b0, b1);
                    mma_bf16(s[q4 * 2 + 1], qf[ks], b2, b3);
                }
            }
            const int key0 = key_base + (lane & 3) * 2;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = key0 + nt * 8 + (c & 1);
                    const int p = (c >> 1) ? pb : pa;
                    const bool ok = j <= p && (window <= 0 || j > p - window);
                    const float v = ok ? s[nt][c] * scale_log2 : -INFINITY;
                    s[nt][c] = v;
                    mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
            float corr[2], base[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const float m_new = fmaxf(m[hh], quad_max(mx[hh]));
                base[hh] = (m_new == -INFINITY) ? 0.f : m_new;
                corr[hh] = exp2f(m[hh] - base[hh]);
                m[hh] = m_new;
            }
            float rs[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
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
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dn = 0; dn < DN; dn += 2) {
                    const int key = kk * 16 + (mi & 1) * 8 + mr;
                    const int chunk = dn + (mi >> 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vt + key * RB + chunk * 16, b0, b1, b2, b3);
                    mma_bf16(o[dn], pf, b0, b1);
                    mma_bf16(o[dn + 1], pf, b2, b3);
                }
            }
        }
        __syncthreads();                             // the stage may be overwritten now
    }
    cp_async_wait<0>();
    if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);
    const float inv_a = l[0] > 0.f ? 1.f / l[0] : 0.f, inv_b = l[1] > 0.f ? 1.f / l[1] : 0.f;
    const int c0 = (lane & 3) * 2;
#pragma unroll
    for (int dn = 0; dn < DN; ++dn) {
        if (ra < r_end)
            *(uint32_t*)(out + ((long long)(row0 + ra) * nq + h) * D + dn * 8 + c0) =
                pack_bf16(o[dn][0] * inv_a, o[dn][1] * inv_a);
        if (rb < r_end)
            *(uint32_t*)(out + ((long long)(row0 + rb) * nq + h) * D + dn * 8 + c0) =
                pack_bf16(o[dn][2] * inv_b, o[dn][3] * inv_b);
    }
}

template <int D>
int launch_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, const int* cu_q,
                   const int* kv_len, const int* block_table, int max_blocks, int num_pages,
                   int page_size, int n_entries, int total_q_tiles, int nq, int nkv, int window,
                   float scale, int skip_single, int* err, cudaStream_t st) {
    constexpr int smem = 4 * BKV * Tile<D>::ROW_BYTES;
    auto kern = paged_prefill_attn_kernel<D>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    dim3 grid(nq, total_q_tiles);
    kern<<<grid, THREADS, smem, st>>>((const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                                      (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_q,
                                      kv_len, block_table, max_blocks, num_pages, page_size, n_entries,
                                      nq, nkv, window, scale * 1.4426950408889634f, skip_single, err);
    return crane_launch_status();
}
}  // namespace

// Every head size is compiled as an object of its own from this file (the build passes
// CRANE_HEAD_SIZE), in parallel; the object without it holds the entry points.
#define CRANE_CAT2(a, b) a##b
#define CRANE_CAT(a, b) CRANE_CAT2(a, b)
#define CRANE_PREFILL_LAUNCHER_ARGS                                                                    \
    const void *q, void *out, const void *k_pool, const void *v_pool, const int *cu_q, const int *kv_len, \
        const int *block_table, int max_blocks, int num_pages, int page_size, int n_entries,            \
        int total_q_tiles, int nq, int nkv, int window, float scale, int skip_single, int *err,         \
        cudaStream_t st
#ifdef CRANE_HEAD_SIZE
extern "C" int CRANE_CAT(crane_prefill_launch_d, CRANE_HEAD_SIZE)(CRANE_PREFILL_LAUNCHER_ARGS) {
    return launch_prefill<CRANE_HEAD_SIZE>(q, out, k_pool, v_pool, cu_q, kv_len, block_table, max_blocks,
                                           num_pages, page_size, n_entries, total_q_tiles, nq, nkv, window,
                                           scale, skip_single, err, st);
}
#else
#ifdef CRANE_HEAD_SIZE_LIST          // the head sizes linked into this library (see attention_decode.cu)
#define CRANE_PREFILL_HEAD_SIZES(X) CRANE_HEAD_SIZE_LIST(X)
#else
#define CRANE_PREFILL_HEAD_SIZES(X) X(16) X(32) X(48) X(64) X(80) X(96) X(112) X(128) X(160) X(192) X(256)
#endif
#define DECLARE(DD) extern "C" int crane_prefill_launch_d##DD(CRANE_PREFILL_LAUNCHER_ARGS);
CRANE_PREFILL_HEAD_SIZES(DECLARE)
#undef DECLARE

CRANE_API int crane_paged_prefill_attention_supports(int d, int nq, int nkv) {
    if (nkv <= 0 || nq % nkv != 0) return 0;
#define IS(DD) if (d == DD) return 1;
    CRANE_PREFILL_HEAD_SIZES(IS)
#undef IS
    return 0;
}

// total_q_tiles: sum over the entries of ceil(q_len / 64) (an upper bound will do: tiles beyond
// the real ones do nothing).  skip_single != 0: entries of exactly one token are left out (they
// count no tile either); their rows of `out` are for the decode kernel to write.
CRANE_API int crane_paged_prefill_attention(const void* q, void* out, const void* k_pool,
                                            const void* v_pool, const int* cu_q, const int* kv_len,
                                            const int* block_table, int max_blocks, int num_pages,
                                            int page_size, int n_entries, int total_q_tiles, int nq,
                                            int nkv, int d, int window, float scale, int skip_single,
                                            int* err, cudaStream_t st) {
    if (n_entries <= 0 || total_q_tiles <= 0) return 0;
    if (!crane_paged_prefill_attention_supports(d, nq, nkv)) return (int)cudaErrorInvalidValue;
#define CASE(DD)                                                                                      \
    case DD:                                                                                          \
        return crane_prefill_launch_d##DD(q, out, k_pool, v_pool, cu_q, kv_len, block_table, max_blocks, \
                                          num_pages, page_size, n_entries, total_q_tiles, nq, nkv,      \
                                          window, scale, skip_single, err, st);
    switch (d) { CRANE_PREFILL_HEAD_SIZES(CASE) }
#undef CASE
    return (int)cudaErrorInvalidValue;
}
#endif  // CRANE_HEAD_SIZE
