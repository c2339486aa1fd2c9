// Attention over the paged cache on the FP32 cores, for any batch of prompt
// portions and single decoded tokens and any head size that is a multiple of
// two up to 256.  One warp per (token, query head): the token at position p of
// request e attends the keys of positions max(0, p - window + 1) .. p of the
// same request, found through the request's block table.  Scores, softmax
// statistics and the weighted sum are float whatever the storage type.
//
// scores = q k^T / sqrt(d), causal j <= p, softmax over the last dimension,
// query head h reads kv head h / (nq / nkv):
// crane-core/src/models/hunyuan_dense/modeling.rs:572-636, 1012-1033.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAXD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simt_kernel(const T* __restrict__ q, T* __restrict__ out,
                            const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                            const int* __restrict__ positions, const int* __restrict__ tok_entry,
                            const int* __restrict__ block_table, int max_blocks, int num_pages,
                            int page_size, int n_tokens, int nq, int nkv, int d, int window,
                            float scale, int* err) {
    __shared__ float q_s[WARPS][MAXD];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * WARPS + wib;
    if (warp >= (long long)n_tokens * nq) return;
    const int t = (int)(warp / nq), h = (int)(warp % nq);
    const int g = h / (nq / nkv);
    const int pos = positions[t];
    if (tok_entry[t] < 0) return;                 // a row that pads the step: it attends to nothing
    const int* table = block_table + (long long)tok_entry[t] * max_blocks;
    const T* qp = q + ((long long)t * nq + h) * d;
    for (int c = lane; c < d; c += 32) q_s[wib][c] = to_f32(qp[c]);
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    constexpr int NACC = MAXD / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool bad = false;

    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        float s = -INFINITY;
        long long row = -1;                       // element offset of this lane's key/value row
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad = true;
            } else {
                row = (((long long)page * nkv + g) * page_size + j % page_size) * d;
                const T* kp = k_pool + row;
                float dot = 0.f;
                for (int c = 0; c < d; ++c) dot = fmaf(q_s[wib][c], to_f32(kp[c]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;         // every key of this chunk was unreadable
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        const int cnt = min(32, pos - base + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (rj < 0) continue;
            const T* vp = v_pool + rj;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int c = lane + 32 * i;
                if (c < d) acc[i] = fmaf(pj, to_f32(vp[c]), acc[i]);
            }
        }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* op = out + ((long long)t * nq + h) * d;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int c = lane + 32 * i;
        if (c < d) op[c] = from_f32<T>(acc[i] * inv);
    }
}
}  // namespace

CRANE_API int crane_paged_attention_simt(int dtype, const void* q, void* out, const void* k_pool,
                                         const void* v_pool, const int* positions,
                                         const int* tok_entry, const int* block_table,
                                         int max_blocks, int num_pages, int page_size,
                                         int n_tokens, int nq, int nkv, int d, int window,
                                         float scale, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (d > MAXD || d <= 0 || nkv <= 0 || nq % nkv != 0) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)n_tokens * nq;
    const int blocks = (int)((warps + WARPS - 1) / WARPS);
    if (dtype == 0)
        paged_attention_simt_kernel<float><<<blocks, WARPS * 32, 0, st>>>(
            (const float*)q, (float*)out, (const float*)k_pool, (const float*)v_pool, positions,
            tok_entry, block_table, max_blocks, num_pages, page_size, n_tokens, nq, nkv, d, window,
            scale, err);
    else
        paged_attention_simt_kernel<__nv_bfloat16><<<blocks, WARPS * 32, 0, st>>>(
            (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, positions, tok_entry, block_table, max_blocks, num_pages,
            page_size, n_tokens, nq, nkv, d, window, scale, err);
    return crane_launch_status();
}
