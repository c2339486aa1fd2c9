// Memory-bound kernels of a decoder step: embedding gather, residual-add +
// RMSNorm, rotary encoding + per-head RMSNorm + write of K/V into cache pages,
// SiLU-gated product.  All arithmetic in 32-bit; T is the storage type of
// activations, weights and cache (float or bf16).  The residual stream itself
// is always float.
//
// Formulas: RMSNorm y = x * rsqrt(mean(x^2) + eps) * w
// (crane-core/kernels/fused_ops.cu:45-51); SiLU-mul silu(g) * u with
// silu(x) = x / (1 + exp(-x)) (fused_ops.cu:39-42, 112-130); rotary encoding
// in the contiguous-halves convention, applied before the per-head norm
// (crane-core/src/models/hunyuan_dense/modeling.rs:541-555).
#include "common.cuh"

int g_crane_pdl = 1;

CRANE_API void crane_set_pdl(int on) { g_crane_pdl = on ? 1 : 0; }

__device__ __forceinline__ float2 ld2(const float* p) { return *(const float2*)p; }
__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*(const __nv_bfloat162*)p);
}
__device__ __forceinline__ void st2(float* p, float a, float b) { *(float2*)p = make_float2(a, b); }
__device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) {
    *(__nv_bfloat162*)p = __floats2bfloat162_rn(a, b);
}

// A GEMM result is either one tensor of T or `n_parts` float partial sums
// (split-K), laid out [part][row][col]; readers add the partials in a fixed
// order and round once to T, so that both forms give the same value.
template <typename T>
struct GemmOut {
    const T* whole;
    const float* parts;
    int n_parts;
    long long part_stride;
    // The partial sums are fetched eight at a time (all loads in flight together) and added in
    // slice order, so the sum is the same as a one-by-one loop's.
    __device__ __forceinline__ float load(long long idx) const {
        if (parts == nullptr) return to_f32(whole[idx]);
        float s = 0.f;
        for (int i = 0; i < n_parts; i += 8) {
            float p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                p[j] = (i + j < n_parts) ? parts[(long long)(i + j) * part_stride + idx] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) s += p[j];
        }
        return to_f32(from_f32<T>(s));
    }
    // two neighbours at once; idx even and the tensors' rows evenly long
    __device__ __forceinline__ float2 load2(long long idx) const {
        if (parts == nullptr) return ld2(whole + idx);
        float2 s = make_float2(0.f, 0.f);
        for (int i = 0; i < n_parts; i += 8) {
            float2 p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                p[j] = (i + j < n_parts) ? *(const float2*)(parts + (long long)(i + j) * part_stride + idx)
                                         : make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s.x += p[j].x;
                s.y += p[j].y;
            }
        }
        return make_float2(to_f32(from_f32<T>(s.x)), to_f32(from_f32<T>(s.y)));
    }
};

// ---------------------------------------------------------------- embedding
// A token id <= -2 stands for "row (-id - 2) of `deferred`": a token that an
// earlier launch on this stream sampled and the host has not seen yet.
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                    float* __restrict__ x, int hidden, int vocab,
                                    const int* __restrict__ deferred, int n_deferred, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok <= -2 && deferred != nullptr && -tok - 2 < n_deferred) tok = deferred[-tok - 2];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_TOKEN_RANGE);
        tok = 0;
    }
    const T* src = table + (long long)tok * hidden;
    float* dst = x + (long long)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]);
}

// ------------------------------------------------------ residual + RMSNorm
// x[row] += delta[row] (if any); out[r] = rmsnorm(x[row]) * w.
// rows == nullptr: row = r = blockIdx.x, x is updated in place.
// rows != nullptr: row = rows[r]; x is left untouched (used for the final norm
// over the wanted positions only).
// A thread keeps its up to PER elements of the row in registers between the
// sum of squares and the scaling, so the row is read once.
// (Up to 1024 threads: the registers of a thread are bounded to what such a block can have.  Rows
// of more than 8192 elements, 16 or 32 per thread, fetch the norm's weights when they scale.)
template <typename T, int PER>
__global__ void __launch_bounds__(1024)
add_rmsnorm_kernel(float* __restrict__ x, GemmOut<T> delta, int has_delta,
                   const float* __restrict__ w, const int* __restrict__ rows,
                   T* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    constexpr bool EARLY_W = PER <= 8;
    const int r = blockIdx.x;
    const int row = rows ? rows[r] : r;          // written by the host's copy, long before
    float* xr = x + (long long)row * hidden;
    const long long dbase = (long long)row * hidden;
    const bool write_x = (rows == nullptr) && has_delta;
    float v[PER], wv[EARLY_W ? PER : 1];
    float ss = 0.f;
    pdl_launch_dependents();
    if (EARLY_W) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {             // the norm's weight depends on no earlier kernel
            const int c = threadIdx.x + k * blockDim.x;
            wv[k] = c < hidden ? w[c] : 0.f;
        }
    }
    pdl_wait();
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = c < hidden ? xr[c] : 0.f;
    }
    if (has_delta) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < hidden) v[k] += delta.load(dbase + c);
        }
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (write_x && c < hidden) xr[c] = v[k];
        ss += v[k] * v[k];
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    T* o = out + (long long)r * hidden;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < hidden) o[c] = from_f32<T>(v[k] * rstd * (EARLY_W ? wv[k] : w[c]));
    }
}

// The same, two neighbouring elements per step (rows of even length).
template <typename T, int PER>
__global__ void __launch_bounds__(PER <= 2 ? 512 : 1024) add_rmsnorm2_kernel(float* __restrict__ x, GemmOut<T> delta, int has_delta,
                                    const float* __restrict__ w, const int* __restrict__ rows,
                                    T* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int row = rows ? rows[r] : r;
    float* xr = x + (long long)row * hidden;
    const long long dbase = (long long)row * hidden;
    const bool write_x = (rows == nullptr) && has_delta;
    float2 v[PER], wv[PER];
    float ss = 0.f;
    pdl_launch_dependents();
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = 2 * (threadIdx.x + k * blockDim.x);
        wv[k] = c < hidden ? ld2(w + c) : make_float2(0.f, 0.f);
    }
    pdl_wait();
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = 2 * (threadIdx.x + k * blockDim.x);
        v[k] = c < hidden ? ld2(xr + c) : make_float2(0.f, 0.f);
    }
    if (has_delta) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int c = 2 * (threadIdx.x + k * blockDim.x);
            if (c < hidden) {
                const float2 d = delta.load2(dbase + c);
                v[k].x += d.x;
                v[k].y += d.y;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = 2 * (threadIdx.x + k * blockDim.x);
        if (write_x && c < hidden) st2(xr + c, v[k].x, v[k].y);
        ss += v[k].x * v[k].x + v[k].y * v[k].y;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    T* o = out + (long long)r * hidden;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int c = 2 * (threadIdx.x + k * blockDim.x);
        if (c < hidden) st2(o + c, v[k].x * rstd * wv[k].x, v[k].y * rstd * wv[k].y);
    }
}

// 8 neighbouring elements at once (16-byte aligned): 32 bytes of float or 16 bytes of bf16
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&q;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 q;
    __nv_bfloat162* h = (__nv_bfloat162*)&q;
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *(uint4*)p = q;
}

// Many rows: a warp per row and no block-wide barrier.  A lane owns CH pieces of 8
// neighbouring elements (piece c at column (c * 32 + lane) * 8), all of whose loads are in
// flight together; the sum of squares goes around the warp by shuffles.  The norm's weights are
// fetched before the wait for the kernel before (2048 x 2048 from DRAM: 13.1 -> 11.1 us).  For a
// delta that is one tensor (not partial sums) and rows of CH * 256 elements.
template <typename T, int CH>
__global__ void __launch_bounds__(256) add_rmsnorm_warp_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                               const float* __restrict__ w, T* __restrict__ out,
                                                               int n_rows, float eps) {
    constexpr int HIDDEN = CH * 256;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_launch_dependents();
    // the weights depend on no earlier kernel: fetched before the wait
    float wv[CH][8];
#pragma unroll
    for (int c = 0; c < CH; ++c) load8(w + (c * 32 + lane) * 8, wv[c]);
    pdl_wait();
    if (row >= n_rows) return;
    float* xr = x + (long long)row * HIDDEN;
    float v[CH][8];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int col = (c * 32 + lane) * 8;
        const float4 a = *(const float4*)(xr + col), b = *(const float4*)(xr + col + 4);
        v[c][0] = a.x; v[c][1] = a.y; v[c][2] = a.z; v[c][3] = a.w;
        v[c][4] = b.x; v[c][5] = b.y; v[c][6] = b.z; v[c][7] = b.w;
    }
    if (delta != nullptr) {
        const T* dr = delta + (long long)row * HIDDEN;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int col = (c * 32 + lane) * 8;
            float d[8];
            load8(dr + col, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[c][j] += d[j];
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int col = (c * 32 + lane) * 8;
            *(float4*)(xr + col) = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
            *(float4*)(xr + col + 4) = make_float4(v[c][4], v[c][5], v[c][6], v[c][7]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
    const float rstd = rsqrtf(warp_sum(ss) / (float)HIDDEN + eps);
    T* o = out + (long long)row * HIDDEN;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int col = (c * 32 + lane) * 8;
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = v[c][j] * rstd * wv[c][j];
        store8(o + col, y);
    }
}

// Few rows (a decode step): a row is shared by a cluster of CL CTAs, each with its
// piece of the columns, so that CL times as many SMs fetch the row and its partial
// sums.  Every CTA sends its sum of squares to all CTAs of the cluster through
// distributed shared memory; after one cluster barrier each adds the CL values up in
// rank order (so all get the same total) and finishes its piece.
template <typename T, int CL>
__global__ void __launch_bounds__(512) add_rmsnorm_cluster_kernel(float* __restrict__ x, GemmOut<T> delta,
                                                                  int has_delta, const float* __restrict__ w,
                                                                  T* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    __shared__ float sums[CL];
    const int rank = blockIdx.x;                  // cluster (CL, 1, 1): the rank is the x index
    const int row = blockIdx.y;
    const int piece = hidden / CL;                // even, checked by the host
    const int c = rank * piece + 2 * threadIdx.x;
    const bool mine = 2 * (int)threadIdx.x < piece;
    float* xr = x + (long long)row * hidden;
    pdl_launch_dependents();
    const float2 wv = mine ? ld2(w + c) : make_float2(0.f, 0.f);
    pdl_wait();
    float2 v = mine ? ld2(xr + c) : make_float2(0.f, 0.f);
    if (has_delta && mine) {
        const float2 d = delta.load2((long long)row * hidden + c);
        v.x += d.x;
        v.y += d.y;
        st2(xr + c, v.x, v.y);
    }
    const float ss = block_sum(v.x * v.x + v.y * v.y, scratch);
    if (threadIdx.x < CL) {
        // my sum goes into slot `rank` of CTA threadIdx.x
        uint32_t local = (uint32_t)__cvta_generic_to_shared(&sums[rank]), remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(threadIdx.x));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(ss) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < CL; ++i) total += sums[i];
    const float rstd = rsqrtf(total / (float)hidden + eps);
    if (mine) st2(out + (long long)row * hidden + c, v.x * rstd * wv.x, v.y * rstd * wv.y);
}

// ------------------------------------- rotary + per-head norm + cache write
// One warp per (token, head).  Heads 0..nq-1 are queries, then nkv keys, then
// nkv values (values are only copied).  `qkv` rows hold [q | k | v]; with
// has_kv == 0 they hold q alone (a layer that reads another layer's cache).
template <typename T, bool PAIRS>
__global__ void rope_norm_cache_kernel(GemmOut<T> qkv, int qkv_stride,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ tok_entry,
                                       const int* __restrict__ block_table, int max_blocks,
                                       const float* __restrict__ cos_tab,
                                       const float* __restrict__ sin_tab, int table_len,
                                       const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, float eps,
                                       T* __restrict__ q_out, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, int num_pages, int page_size,
                                       int n_tokens, int nq, int nkv, int d, int has_kv,
                                       int rotary, RopeParams rp, int general, int* err) {
    pdl_launch_dependents();
    const int heads = nq + (has_kv ? 2 * nkv : 0);
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const bool in = warp < n_tokens * heads;
    const int t = in ? warp / heads : 0, h = in ? warp % heads : 0;
    // the step's positions and block tables were written before the step began: they are looked up
    // before the wait for the product that makes q, k and v
    const int pos = positions[t];
    int e = -1, page = -1;
    if (in && h >= nq) {
        e = tok_entry[t];
        if (e >= 0) page = block_table[(long long)e * max_blocks + pos / page_size];
    }
    pdl_wait();
    if (!in) return;
    const int half = d >> 1;
    const long long src = (long long)t * qkv_stride + (long long)h * d;   // q,k,v are consecutive

    T* dst;
    const float* nw = nullptr;
    bool rotate = rotary != 0;
    if (h < nq) {
        dst = q_out + ((long long)t * nq + h) * d;
        nw = q_norm_w;
    } else {
        if (e < 0) return;                         // a row that pads the step: it has no place in a cache
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
            return;
        }
        const bool is_v = h >= nq + nkv;
        const int g = is_v ? h - nq - nkv : h - nq;
        T* pool = is_v ? v_pool : k_pool;
        dst = pool + (((long long)page * nkv + g) * page_size + pos % page_size) * d;
        if (is_v) {
            if (PAIRS) {
                for (int c = 2 * lane; c < d; c += 64) {
                    const float2 x = qkv.load2(src + c);
                    st2(dst + c, x.x, x.y);
                }
            } else {
                for (int c = lane; c < d; c += 32) dst[c] = from_f32<T>(qkv.load(src + c));
            }
            return;
        }
        nw = k_norm_w;
    }
    if (rotate && (pos < 0 || pos >= table_len)) {
        if (lane == 0) atomicOr(err, CRANE_ERR_POSITION_RANGE);
        rotate = false;
    }
    if (general) {
        // another pairing, a partly rotated head, the norm first or (1 + w) weights: element by element
        rope_norm_general<8>(rp, d, pos, rotate, cos_tab, sin_tab, nw, eps, lane,
                             [&](int e) { return qkv.load(src + e); },
                             [&](int e, float v) { dst[e] = from_f32<T>(v); });
        return;
    }
    if (PAIRS) {
        // each lane owns j, j + 1 and their partners j + d/2, j + 1 + d/2 for j = 2 lane, 2 lane + 64, ...
        constexpr int MAXP2 = 4;                  // d <= 512
        float2 a2[MAXP2], b2[MAXP2];
        float ss2 = 0.f;
#pragma unroll
        for (int i = 0; i < MAXP2; ++i) {
            const int j = 2 * lane + 64 * i;
            a2[i] = b2[i] = make_float2(0.f, 0.f);
            if (j < half) {
                const float2 x1 = qkv.load2(src + j), x2 = qkv.load2(src + j + half);
                if (rotate) {
                    const float2 c = ld2(cos_tab + (long long)pos * half + j);
                    const float2 sn = ld2(sin_tab + (long long)pos * half + j);
                    a2[i] = make_float2(x1.x * c.x - x2.x * sn.x, x1.y * c.y - x2.y * sn.y);
                    b2[i] = make_float2(x2.x * c.x + x1.x * sn.x, x2.y * c.y + x1.y * sn.y);
                } else {
                    a2[i] = x1;
                    b2[i] = x2;
                }
                ss2 += a2[i].x * a2[i].x + a2[i].y * a2[i].y + b2[i].x * b2[i].x + b2[i].y * b2[i].y;
            }
        }
        float rstd2 = 1.f;
        if (nw != nullptr) rstd2 = rsqrtf(warp_sum(ss2) / (float)d + eps);
#pragma unroll
        for (int i = 0; i < MAXP2; ++i) {
            const int j = 2 * lane + 64 * i;
            if (j < half) {
                float2 y1 = a2[i], y2 = b2[i];
                if (nw != nullptr) {
                    const float2 w1 = ld2(nw + j), w2 = ld2(nw + j + half);
                    y1 = make_float2(y1.x * rstd2 * w1.x, y1.y * rstd2 * w1.y);
                    y2 = make_float2(y2.x * rstd2 * w2.x, y2.y * rstd2 * w2.y);
                }
                st2(dst + j, y1.x, y1.y);
                st2(dst + j + half, y2.x, y2.y);
            }
        }
        return;
    }
    // each lane owns the pairs (j, j + d/2) for j = lane, lane + 32, ...
    constexpr int MAXP = 8;                       // d <= 512
    float a[MAXP], b[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int j = lane + 32 * i;
        a[i] = b[i] = 0.f;
        if (j < half) {
            const float x1 = qkv.load(src + j), x2 = qkv.load(src + j + half);
            if (rotate) {
                const float c = cos_tab[(long long)pos * half + j];
                const float s = sin_tab[(long long)pos * half + j];
                a[i] = x1 * c - x2 * s;
                b[i] = x2 * c + x1 * s;
            } else {
                a[i] = x1;
                b[i] = x2;
            }
            ss += a[i] * a[i] + b[i] * b[i];
        }
    }
    float rstd = 1.f;
    if (nw != nullptr) {
        ss = warp_sum(ss);
        rstd = rsqrtf(ss / (float)d + eps);
    }
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int j = lane + 32 * i;
        if (j < half) {
            float y1 = a[i], y2 = b[i];
            if (nw != nullptr) {
                y1 = y1 * rstd * nw[j];
                y2 = y2 * rstd * nw[j + half];
            }
            dst[j] = from_f32<T>(y1);
            dst[j + half] = from_f32<T>(y2);
        }
    }
}

// The same for whole bf16 rows of head size 128, eight lanes per (token, head): a
// lane owns eight neighbours of the first half and their partners in the second
// half (16-byte loads and stores), four heads per warp.
__global__ void rope_norm_cache_d128_kernel(const __nv_bfloat16* __restrict__ qkv, int qkv_stride,
                                            const int* __restrict__ positions,
                                            const int* __restrict__ tok_entry,
                                            const int* __restrict__ block_table, int max_blocks,
                                            const float* __restrict__ cos_tab,
                                            const float* __restrict__ sin_tab, int table_len,
                                            const float* __restrict__ q_norm_w,
                                            const float* __restrict__ k_norm_w, float eps,
                                            __nv_bfloat16* __restrict__ q_out,
                                            __nv_bfloat16* __restrict__ k_pool,
                                            __nv_bfloat16* __restrict__ v_pool, int num_pages,
                                            int page_size, int n_tokens, int nq, int nkv, int has_kv,
                                            int rotary, int* err) {
    constexpr int D = 128, HALF = 64;
    pdl_launch_dependents();
    // Positions, block tables, the cosine and sine tables and the norm weights were written before
    // the step began: they are fetched before the wait for the product that makes q, k and v, so
    // that after it only the rows themselves are on the way.
    const int heads = nq + (has_kv ? 2 * nkv : 0);
    const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int sub = threadIdx.x & 7;                         // which eighth of a half
    const bool live = item < (long long)n_tokens * heads;
    const int t = live ? (int)(item / heads) : 0, h = live ? (int)(item % heads) : 0;
    const int pos = positions[t];
    const __nv_bfloat16* src = qkv + (long long)t * qkv_stride + (long long)h * D;
    __nv_bfloat16* dst = nullptr;
    const float* nw = nullptr;
    bool is_v = false;
    if (live) {
        if (h < nq) {
            dst = q_out + ((long long)t * nq + h) * D;
            nw = q_norm_w;
        } else {
            // a negative entry: a row that pads the step; it has no place in a cache, dst stays null
            const int e = tok_entry[t];
            const int page = e < 0 ? -1 : block_table[(long long)e * max_blocks + pos / page_size];
            if (e >= 0 && (page < 0 || page >= num_pages)) {
                if (sub == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
            } else if (e >= 0) {
                is_v = h >= nq + nkv;
                const int g = is_v ? h - nq - nkv : h - nq;
                dst = (is_v ? v_pool : k_pool) + (((long long)page * nkv + g) * page_size + pos % page_size) * D;
                nw = is_v ? nullptr : k_norm_w;
            }
        }
    }
    bool rotate = rotary != 0 && !is_v;
    if (live && rotate && (pos < 0 || pos >= table_len)) {
        if (sub == 0) atomicOr(err, CRANE_ERR_POSITION_RANGE);
        rotate = false;
    }
    float c[8], sn[8], wa[8], wb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = sn[i] = wa[i] = wb[i] = 0.f;
    if (live && rotate) {
        const float4* c4 = (const float4*)(cos_tab + (long long)pos * HALF + 8 * sub);
        const float4* s4 = (const float4*)(sin_tab + (long long)pos * HALF + 8 * sub);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    if (nw != nullptr) {
        const float4* w4 = (const float4*)(nw + 8 * sub);
        const float4* v4 = (const float4*)(nw + HALF + 8 * sub);
        const float4 w0 = w4[0], w1 = w4[1], v0 = v4[0], v1 = v4[1];
        wa[0] = w0.x; wa[1] = w0.y; wa[2] = w0.z; wa[3] = w0.w; wa[4] = w1.x; wa[5] = w1.y; wa[6] = w1.z; wa[7] = w1.w;
        wb[0] = v0.x; wb[1] = v0.y; wb[2] = v0.z; wb[3] = v0.w; wb[4] = v1.x; wb[5] = v1.y; wb[6] = v1.z; wb[7] = v1.w;
    }
    pdl_wait();
    float a[8], b[8];
    {
        uint4 ra = make_uint4(0, 0, 0, 0), rb = ra;
        if (live) {
            ra = *(const uint4*)(src + 8 * sub);
            rb = *(const uint4*)(src + HALF + 8 * sub);
        }
        const __nv_bfloat162* pa = (const __nv_bfloat162*)&ra;
        const __nv_bfloat162* pb = (const __nv_bfloat162*)&rb;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
            a[2 * i] = fa.x; a[2 * i + 1] = fa.y;
            b[2 * i] = fb.x; b[2 * i + 1] = fb.y;
        }
    }
    if (live && rotate) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x1 = a[i], x2 = b[i];
            a[i] = x1 * c[i] - x2 * sn[i];
            b[i] = x2 * c[i] + x1 * sn[i];
        }
    }
    {
        // every lane takes part in the shuffles, whatever its head is
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (nw != nullptr) {
            const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[i] = a[i] * rstd * wa[i];
                b[i] = b[i] * rstd * wb[i];
            }
        }
    }
    if (dst != nullptr) {
        uint4 oa, ob;
        __nv_bfloat162* qa = (__nv_bfloat162*)&oa;
        __nv_bfloat162* qb = (__nv_bfloat162*)&ob;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
            qb[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
        }
        *(uint4*)(dst + 8 * sub) = oa;
        *(uint4*)(dst + HALF + 8 * sub) = ob;
    }
}

// ------------------------------------------------------------ SiLU(g) * u
// gu rows hold [gate (inter) | up (inter)], or, `blocked`, blocks of 16 gate
// columns followed by the 16 up columns of the same features.
template <typename T>
__global__ void silu_mul_kernel(GemmOut<T> gu, T* __restrict__ out, long long n_rows, int inter,
                                int blocked) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * inter) return;
    const long long r = i / inter;
    const int c = (int)(i % inter);
    const int gc = blocked ? (c >> 4) * 32 + (c & 15) : c;
    const int uc = blocked ? gc + 16 : inter + c;
    const float g = gu.load(r * 2 * inter + gc);
    const float u = gu.load(r * 2 * inter + uc);
    out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

// The same for whole bf16 rows, eight neighbours per thread (inter % 8 == 0).
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu,
                                       __nv_bfloat16* __restrict__ out, int inter, int blocked) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= inter) return;
    const long long r = blockIdx.y;
    const int gc = blocked ? (c >> 4) * 32 + (c & 15) : c;
    const int uc = blocked ? gc + 16 : inter + c;
    const uint4 g4 = *(const uint4*)(gu + r * 2 * inter + gc);
    const uint4 u4 = *(const uint4*)(gu + r * 2 * inter + uc);
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&g4;
    const __nv_bfloat162* u2 = (const __nv_bfloat162*)&u4;
    uint4 o4;
    __nv_bfloat162* o2 = (__nv_bfloat162*)&o4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        o2[i] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
    }
    *(uint4*)(out + r * inter + c) = o4;
}

// a T tensor to float (logits of a bf16 head, test helpers)
template <typename T>
__global__ void to_float_kernel(const T* __restrict__ in, float* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = to_f32(in[i]);
}

// out[r, c] = sum over the split-K partial sums parts[i][r][c], in slice order, kept in float (the
// float logits of a head whose product was computed in slices of the inner dimension)
__global__ void sum_parts_kernel(const float* __restrict__ parts, int n_parts, long long part_stride,
                                 long long row_pitch, float* __restrict__ out, long long out_pitch,
                                 int rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const long long r = i / cols, c = i % cols;
    const float* p = parts + r * row_pitch + c;
    float s = 0.f;
    for (int k = 0; k < n_parts; k += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (k + j < n_parts) ? p[(long long)(k + j) * part_stride] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[j];
    }
    out[r * out_pitch + c] = s;
}

static bool norm_cluster_on() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("CRANE_NORM_CLUSTER");
        on = (v == nullptr || v[0] != '0') ? 1 : 0;
    }
    return on == 1;
}

// ------------------------------------------------------------------ C ABI
// dtype: 0 = float, 1 = bf16.  Every function returns the CUDA launch status.
#define DISPATCH_T(dtype, ...)                                   \
    if ((dtype) == 0) { using T = float; __VA_ARGS__; }          \
    else { using T = __nv_bfloat16; __VA_ARGS__; }

CRANE_API int crane_embed_gather(int dtype, const int* tokens, const void* table, float* x,
                                 int n_tokens, int hidden, int vocab, const int* deferred,
                                 int n_deferred, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    DISPATCH_T(dtype, return crane_launch(embed_gather_kernel<T>, dim3(n_tokens), dim3(256), 0, st, tokens,
                                          (const T*)table, x, hidden, vocab, deferred, n_deferred, err));
}

CRANE_API int crane_add_rmsnorm(int dtype, float* x, const void* delta, const float* delta_parts,
                                int n_parts, long long part_stride, const float* w,
                                const int* rows, void* out, int n_rows, int hidden, float eps,
                                cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const int has_delta = (delta != nullptr || delta_parts != nullptr) ? 1 : 0;
    // 4 elements per thread up to 4096 wide, then more per thread at 1024 threads
    int per = 4;
    while (per < 32 && (hidden + per - 1) / per > 1024) per *= 2;
    if ((hidden + per - 1) / per > 1024) return (int)cudaErrorInvalidValue;    // wider than 32768
    int threads = ((hidden + per - 1) / per + 31) / 32 * 32;
    const bool aligned = ((uintptr_t)x | (uintptr_t)delta | (uintptr_t)delta_parts | (uintptr_t)w |
                          (uintptr_t)out) % 8 == 0 && part_stride % 2 == 0;
    if (rows == nullptr && n_rows <= 64 && aligned && hidden % 16 == 0 && hidden <= 8192 && norm_cluster_on()) {
        // few rows: a cluster of 4 CTAs per row, 8 for long rows
        DISPATCH_T(dtype, {
            GemmOut<T> d{(const T*)delta, delta_parts, n_parts, part_stride};
            if (hidden >= 4096)
                return crane_launch_cluster(add_rmsnorm_cluster_kernel<T, 8>, dim3(8, n_rows),
                                            dim3((hidden / 16 + 31) / 32 * 32), 0, dim3(8, 1, 1), st, x, d,
                                            has_delta, w, (T*)out, hidden, eps);
            return crane_launch_cluster(add_rmsnorm_cluster_kernel<T, 4>, dim3(4, n_rows),
                                        dim3((hidden / 8 + 31) / 32 * 32), 0, dim3(4, 1, 1), st, x, d,
                                        has_delta, w, (T*)out, hidden, eps);
        });
    }
    if (rows == nullptr && n_rows >= 256 && delta_parts == nullptr && hidden % 256 == 0 && hidden <= 2048 &&
        ((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) % 16 == 0) {
        // many rows: a warp per row
        const dim3 g((n_rows + 7) / 8), b(256);
#define WARP_CASE(CH)                                                                                  \
    case CH:                                                                                           \
        DISPATCH_T(dtype, return crane_launch(add_rmsnorm_warp_kernel<T, CH>, g, b, 0, st, x, (const T*)delta, w, \
                                              (T*)out, n_rows, eps));
        switch (hidden / 256) {
            WARP_CASE(1) WARP_CASE(2) WARP_CASE(3) WARP_CASE(4) WARP_CASE(5) WARP_CASE(6) WARP_CASE(7) WARP_CASE(8)
        }
#undef WARP_CASE
    }
    if (hidden % 2 == 0 && hidden <= 8192 && aligned) {
        // pairs of neighbours: 2 or 4 pairs per thread
        const int pp = hidden <= 2048 ? 2 : 4;
        const int th = ((hidden / 2 + pp - 1) / pp + 31) / 32 * 32;
        DISPATCH_T(dtype, {
            GemmOut<T> d{(const T*)delta, delta_parts, n_parts, part_stride};
            if (pp == 2)
                return crane_launch(add_rmsnorm2_kernel<T, 2>, dim3(n_rows), dim3(th), 0, st, x, d, has_delta, w,
                                    rows, (T*)out, hidden, eps);
            return crane_launch(add_rmsnorm2_kernel<T, 4>, dim3(n_rows), dim3(th), 0, st, x, d, has_delta, w,
                                rows, (T*)out, hidden, eps);
        });
    }
    DISPATCH_T(dtype, {
        GemmOut<T> d{(const T*)delta, delta_parts, n_parts, part_stride};
        const dim3 g(n_rows), b(threads);
        if (per == 4)
            return crane_launch(add_rmsnorm_kernel<T, 4>, g, b, 0, st, x, d, has_delta, w, rows, (T*)out, hidden, eps);
        if (per == 8)
            return crane_launch(add_rmsnorm_kernel<T, 8>, g, b, 0, st, x, d, has_delta, w, rows, (T*)out, hidden, eps);
        if (per == 16)
            return crane_launch(add_rmsnorm_kernel<T, 16>, g, b, 0, st, x, d, has_delta, w, rows, (T*)out, hidden, eps);
        return crane_launch(add_rmsnorm_kernel<T, 32>, g, b, 0, st, x, d, has_delta, w, rows, (T*)out, hidden, eps);
    });
}

CRANE_API int crane_rope_norm_cache(int dtype, const void* qkv, const float* qkv_parts, int n_parts,
                                    long long part_stride, int qkv_stride, const int* positions,
                                    const int* tok_entry, const int* block_table, int max_blocks,
                                    const float* cos_tab, const float* sin_tab, int table_len,
                                    const float* q_norm_w, const float* k_norm_w, float eps,
                                    void* q_out, void* k_pool, void* v_pool, int num_pages,
                                    int page_size, int n_tokens, int nq, int nkv, int d, int has_kv,
                                    int rotary, int rotary_dim, int interleaved, int norm_first,
                                    float norm_offset, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (d > 512 || (d & 1)) return (int)cudaErrorInvalidValue;
    if (rotary_dim <= 0) rotary_dim = d;
    if (rotary_dim > d || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
    const RopeParams rp{rotary_dim, interleaved ? 1 : 0, norm_first ? 1 : 0, norm_offset};
    const int general = rope_is_default(rp, d) ? 0 : 1;
    const int heads = nq + (has_kv ? 2 * nkv : 0);
    const long long warps = (long long)n_tokens * heads;
    const int threads = 128;
    const int blocks = (int)((warps * 32 + threads - 1) / threads);
    if (!general && dtype == 1 && d == 128 && qkv != nullptr && qkv_stride % 8 == 0 && n_tokens >= 32 &&
        ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)cos_tab |
         (uintptr_t)sin_tab | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) % 16 == 0) {
        const long long lanes = warps * 8;
        return crane_launch(rope_norm_cache_d128_kernel, dim3((unsigned)((lanes + 255) / 256)), dim3(256), 0, st,
                            (const __nv_bfloat16*)qkv, qkv_stride, positions, tok_entry, block_table,
                            max_blocks, cos_tab, sin_tab, table_len, q_norm_w, k_norm_w, eps,
                            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, num_pages,
                            page_size, n_tokens, nq, nkv, has_kv, rotary, err);
    }
    DISPATCH_T(dtype, {
        GemmOut<T> src{(const T*)qkv, qkv_parts, n_parts, part_stride};
        // two neighbours per load when every row starts on an even element and 8-byte boundary
        const bool pairs = d % 4 == 0 && qkv_stride % 2 == 0 && part_stride % 2 == 0 &&
                           ((uintptr_t)qkv | (uintptr_t)qkv_parts | (uintptr_t)q_out | (uintptr_t)k_pool |
                            (uintptr_t)v_pool | (uintptr_t)cos_tab | (uintptr_t)sin_tab |
                            (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) % 8 == 0;
        if (pairs)
            return crane_launch(rope_norm_cache_kernel<T, true>, dim3(blocks), dim3(threads), 0, st, src,
                                qkv_stride, positions, tok_entry, block_table, max_blocks, cos_tab, sin_tab,
                                table_len, q_norm_w, k_norm_w, eps, (T*)q_out, (T*)k_pool, (T*)v_pool,
                                num_pages, page_size, n_tokens, nq, nkv, d, has_kv, rotary, rp, general, err);
        return crane_launch(rope_norm_cache_kernel<T, false>, dim3(blocks), dim3(threads), 0, st, src,
                            qkv_stride, positions, tok_entry, block_table, max_blocks, cos_tab, sin_tab,
                            table_len, q_norm_w, k_norm_w, eps, (T*)q_out, (T*)k_pool, (T*)v_pool,
                            num_pages, page_size, n_tokens, nq, nkv, d, has_kv, rotary, rp, general, err);
    });
}

CRANE_API int crane_silu_mul(int dtype, const void* gu, const float* gu_parts, int n_parts,
                             long long part_stride, void* out, int n_rows, int inter, int blocked,
                             cudaStream_t st) {
    if (blocked && (inter & 15)) return (int)cudaErrorInvalidValue;
    if (n_rows <= 0) return 0;
    const long long n = (long long)n_rows * inter;
    const int blocks = (int)((n + 255) / 256);
    if (dtype == 1 && gu != nullptr && inter % 8 == 0 && n_rows <= 65535 &&
        ((uintptr_t)gu | (uintptr_t)out) % 16 == 0)
        return crane_launch(silu_mul_bf16x8_kernel, dim3((inter / 8 + 127) / 128, n_rows), dim3(128), 0, st,
                            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, blocked);
    DISPATCH_T(dtype, {
        GemmOut<T> src{(const T*)gu, gu_parts, n_parts, part_stride};
        return crane_launch(silu_mul_kernel<T>, dim3(blocks), dim3(256), 0, st, src, (T*)out,
                            (long long)n_rows, inter, blocked);
    });
}

CRANE_API int crane_to_float(int dtype, const void* in, float* out, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256);
    DISPATCH_T(dtype, (to_float_kernel<T><<<blocks, 256, 0, st>>>((const T*)in, out, n)));
    return crane_launch_status();
}

CRANE_API int crane_sum_parts(const float* parts, int n_parts, long long part_stride, long long row_pitch,
                              float* out, long long out_pitch, int rows, int cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0 || n_parts <= 0) return 0;
    const long long n = (long long)rows * cols;
    return crane_launch(sum_parts_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, parts, n_parts,
                        part_stride, row_pitch, out, out_pitch, rows, cols);
}
