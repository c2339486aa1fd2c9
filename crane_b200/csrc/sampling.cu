// Sampling over float logits [rows, vocab], one block per row, each row with
// its own options: repetition penalty, greedy argmax (ties go to the lowest
// index), Gumbel-max temperature sampling over the whole vocabulary, and
// top-k (k <= 64) with top-p inside the top-k set.
//
// Rules restated from crane-serve/src/engine/sampling.rs: greedy when
// temperature <= 0 (:129-132); seen tokens' logits divided by the penalty if
// >= 0, else multiplied, once per distinct token (:301-327); top-k clamped to
// 64 and top-p evaluated on a softmax over the top-k set, keeping the entries
// whose cumulative probability is <= top_p and the one after them (:202,
// :237-258); argmax(logits / T - log(-log u)), u uniform in [1e-7, 0.999)
// (:288-298).  The uniforms come from a counter-based generator keyed by
// (seed, counter, vocabulary index), so a host restatement reproduces them.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;
constexpr int MAXK = 64;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__device__ __forceinline__ float uniform_at(unsigned long long key, int idx) {
    const unsigned long long x = splitmix64(key ^ ((unsigned long long)idx * 0xD6E8FEB86659FD93ull));
    const float r = (float)(x >> 40) * (1.0f / 16777216.0f);
    return 1e-7f + (0.999f - 1e-7f) * r;
}
__device__ __forceinline__ float gumbel_score(float logit, float inv_t, unsigned long long key,
                                              int idx) {
    return logit * inv_t - logf(-logf(uniform_at(key, idx)));
}

struct Best {
    float v;
    int i;
};
// order: larger value first, then lower index
__device__ __forceinline__ bool better(float v, int i, const Best& b) {
    return v > b.v || (v == b.v && i < b.i);
}
__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (better(ov, oi, b)) { b.v = ov; b.i = oi; }
    }
    return b;
}
__device__ Best block_best(Best b, Best* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    b = warp_best(b);
    __syncthreads();
    if (lane == 0) scratch[warp] = b;
    __syncthreads();
    Best r = (lane < (THREADS >> 5)) ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
    return warp_best(r);
}

__global__ void repetition_penalty_kernel(float* __restrict__ logits, long long row_stride,
                                          int vocab, const int* __restrict__ context,
                                          int ctx_stride, const int* __restrict__ ctx_len,
                                          const float* __restrict__ penalty) {
    const int r = blockIdx.x;
    const float pen = penalty[r];
    if (pen == 1.0f) return;
    const int n = ctx_len[r];
    const int* ctx = context + (long long)r * ctx_stride;
    float* row = logits + (long long)r * row_stride;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int tok = ctx[i];
        if (tok < 0 || tok >= vocab) continue;
        bool first = true;                      // act once per distinct token
        for (int j = 0; j < i; ++j)
            if (ctx[j] == tok) { first = false; break; }
        if (!first) continue;
        const float v = row[tok];
        row[tok] = v >= 0.f ? v / pen : v * pen;
    }
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
              const unsigned long long* __restrict__ counter, int* __restrict__ out) {
    __shared__ Best scratch[THREADS / 32];
    __shared__ float cand_v[MAXK];
    __shared__ int cand_i[MAXK];
    const int r = blockIdx.x;
    const float* row = logits + (long long)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    Best b{-INFINITY, 0x7fffffff};

    if (!(temp > 0.f)) {                                        // greedy
        if ((((uintptr_t)row) & 7) == 0) {
            // pairs of neighbours, four pairs in flight per thread
            const int pairs = vocab >> 1;
            const float2* row2 = (const float2*)row;
            int i = threadIdx.x;
            for (; i + 3 * THREADS < pairs; i += 4 * THREADS) {
                const float2 a = row2[i], c = row2[i + THREADS], d = row2[i + 2 * THREADS],
                             f = row2[i + 3 * THREADS];
                if (better(a.x, 2 * i, b)) { b.v = a.x; b.i = 2 * i; }
                if (better(a.y, 2 * i + 1, b)) { b.v = a.y; b.i = 2 * i + 1; }
                if (better(c.x, 2 * (i + THREADS), b)) { b.v = c.x; b.i = 2 * (i + THREADS); }
                if (better(c.y, 2 * (i + THREADS) + 1, b)) { b.v = c.y; b.i = 2 * (i + THREADS) + 1; }
                if (better(d.x, 2 * (i + 2 * THREADS), b)) { b.v = d.x; b.i = 2 * (i + 2 * THREADS); }
                if (better(d.y, 2 * (i + 2 * THREADS) + 1, b)) { b.v = d.y; b.i = 2 * (i + 2 * THREADS) + 1; }
                if (better(f.x, 2 * (i + 3 * THREADS), b)) { b.v = f.x; b.i = 2 * (i + 3 * THREADS); }
                if (better(f.y, 2 * (i + 3 * THREADS) + 1, b)) { b.v = f.y; b.i = 2 * (i + 3 * THREADS) + 1; }
            }
            for (; i < pairs; i += THREADS) {
                const float2 a = row2[i];
                if (better(a.x, 2 * i, b)) { b.v = a.x; b.i = 2 * i; }
                if (better(a.y, 2 * i + 1, b)) { b.v = a.y; b.i = 2 * i + 1; }
            }
            if ((vocab & 1) && threadIdx.x == 0) {
                const float v = row[vocab - 1];
                if (better(v, vocab - 1, b)) { b.v = v; b.i = vocab - 1; }
            }
        } else {
            for (int i = threadIdx.x; i < vocab; i += THREADS) {
                const float v = row[i];
                if (better(v, i, b)) { b.v = v; b.i = i; }
            }
        }
        b = block_best(b, scratch);
        if (threadIdx.x == 0) out[r] = b.i < vocab ? b.i : 0;
        return;
    }
    const float inv_t = 1.f / temp;
    const unsigned long long key = splitmix64(seed[r] + counter[r] * 0x9E3779B97F4A7C15ull);
    int k = top_k ? top_k[r] : 0;
    const float p = top_p ? top_p[r] : 1.f;
    const bool p_active = p > 0.f && p < 1.f;
    if (k <= 0 && p_active) k = MAXK;
    if (k > MAXK) k = MAXK;
    if (k > vocab) k = vocab;

    if (k <= 0 || (k >= vocab && !p_active)) {                   // whole vocabulary (top-p needs the sorted candidates)
        for (int i = threadIdx.x; i < vocab; i += THREADS) {
            const float v = gumbel_score(row[i], inv_t, key, i);
            if (better(v, i, b)) { b.v = v; b.i = i; }
        }
        b = block_best(b, scratch);
        if (threadIdx.x == 0) out[r] = b.i < vocab ? b.i : 0;
        return;
    }
    // top-k by k passes: each pass finds the best entry that comes after the last pick
    Best last{INFINITY, -1};
    for (int n = 0; n < k; ++n) {
        Best c{-INFINITY, 0x7fffffff};
        for (int i = threadIdx.x; i < vocab; i += THREADS) {
            const float v = row[i];
            const bool after = v < last.v || (v == last.v && i > last.i);
            if (after && better(v, i, c)) { c.v = v; c.i = i; }
        }
        c = block_best(c, scratch);
        if (threadIdx.x == 0) { cand_v[n] = c.v; cand_i[n] = c.i; }
        last = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int keep = k;
        if (p_active) {
            const float mx = cand_v[0] * inv_t;
            float sum = 0.f;
            for (int n = 0; n < k; ++n) sum += expf(cand_v[n] * inv_t - mx);
            float cum = 0.f;
            keep = 1;
            for (int n = 0; n < k; ++n) {
                cum += expf(cand_v[n] * inv_t - mx) / sum;
                if (cum <= p) keep = min(k, n + 2); else break;
            }
        }
        Best w{-INFINITY, 0x7fffffff};
        for (int n = 0; n < keep; ++n) {
            if (cand_i[n] >= vocab) continue;
            const float v = gumbel_score(cand_v[n], inv_t, key, cand_i[n]);
            if (better(v, cand_i[n], w)) { w.v = v; w.i = cand_i[n]; }
        }
        out[r] = w.i < vocab ? w.i : 0;
    }
}
}  // namespace

CRANE_API int crane_repetition_penalty(float* logits, long long row_stride, int rows, int vocab,
                                       const int* context, int ctx_stride, const int* ctx_len,
                                       const float* penalty, cudaStream_t st) {
    if (rows <= 0) return 0;
    repetition_penalty_kernel<<<rows, 128, 0, st>>>(logits, row_stride, vocab, context, ctx_stride,
                                                    ctx_len, penalty);
    return crane_launch_status();
}

// temperature == nullptr: every row greedy.
CRANE_API int crane_sample(const float* logits, long long row_stride, int rows, int vocab,
                           const float* temperature, const int* top_k, const float* top_p,
                           const unsigned long long* seed, const unsigned long long* counter,
                           int* out, cudaStream_t st) {
    if (rows <= 0) return 0;
    sample_kernel<<<rows, THREADS, 0, st>>>(logits, row_stride, vocab, temperature, top_k, top_p,
                                            seed, counter, out);
    return crane_launch_status();
}
