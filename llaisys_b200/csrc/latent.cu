// Row-wise kernels of latent attention: queries, keys and values all pass through low-rank latents, and what a token
// leaves in the cache is one row [latent c (kv_rank) | rotated shared key part (rope_dim)] for all heads together.
//
// Since a head's unrotated key is W_uk[h] c and its value W_uv[h] c, the score q_n . (W_uk[h] c) equals
// (W_uk[h]^T q_n) . c and the head's output is W_uv[h] (sum_t p_t c_t): attention runs over the cached rows themselves,
// as one key/value head that every query head shares, with the query carried into the latent space first and the
// latent result carried into the head's value space afterwards.
//
//  * latent_prep: per token, from the fused down projections: RMS norm (plain weight) of the query latent; RMS norm
//    of the key/value latent; rotation of the shared key part (pairs (2i, 2i+1), angles from float32 tables that
//    already hold any rescaling of frequency and magnitude); the row [c | rotated part] is written densely for the
//    step's attention and, with `append`, into the token's row of the paged cache.  With `halves` the rotated pairs
//    are (i, i + rot/2) instead (here and in the two kernels below).
//  * latent_append: the same rows into the paged cache as a pass of its own (a ring cache is appended to after the
//    step's attention).
//  * head_matmul: y[t, h, :] = x[t, h, :] M[h]  (M [heads, in, out]) with float32 accumulation: the query's unrotated
//    part into the latent space, the latent result into the value space; optional tail: rotation of the `tail`
//    elements that follow x[t, h, :in] into y[t, h, out:]; optional per-(token, head) factor sigmoid(gate[t, h]).
#include "common.cuh"

struct LatentPrepParams {
    const void* proj;         // [T, row_stride]
    int row_stride;
    int q_off, q_rank;        // the query latent's columns
    int kv_off, kv_rank;      // the key/value latent's columns (kv_rank 0: the layer projects none)
    int kr_off, rope_dim;     // the shared key part's columns
    int rot;                  // rotated dimensions (<= rope_dim, even)
    const void* wq;           // [q_rank] norm weight
    const void* wkv;          // [kv_rank]
    float eps;
    const float* cos_t;       // [table_rows, rot / 2]
    const float* sin_t;
    int table_rows;
    const int* tok_pos;
    void* q_out;              // [T, q_rank]
    void* kv_out;             // [T, kv_rank + rope_dim]
    // append
    int append;
    const int* tok_seq;
    const int* seq_start;
    const int* seq_len_before;
    void* pool;               // [pages, 1, LLB_PAGE, kv_rank + rope_dim]
    const int* page_table;
    int table_stride, ring, pinned;
    int* err;
    int halves;               // rotated pairs are (i, i + rot / 2) instead of (2i, 2i + 1)
};

template <typename T, typename TW>
__global__ void __launch_bounds__(256) latent_prep_kernel(LatentPrepParams p) {
    __shared__ float red[8];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int pos = p.tok_pos[t];
    if (p.kv_rank > 0 && p.rot > 0 && (pos < 0 || pos >= p.table_rows)) {
        if (tid == 0) atomicExch(p.err, 2);
        return;
    }
    llb_grid_dependency_sync();
    const T* row = (const T*)p.proj + (size_t)t * p.row_stride;
    // ---- the query latent (q_rank 0: the layer's queries pass through none)
    if (p.q_rank > 0) {
        float ss = 0.f;
        for (int j = tid; j < p.q_rank; j += 256) {
            float v = to_f32(row[p.q_off + j]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[wp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot += red[i];
        const float inv = 1.0f / sqrtf(tot / (float)p.q_rank + p.eps);
        T* qo = (T*)p.q_out + (size_t)t * p.q_rank;
        const TW* w = (const TW*)p.wq;
        for (int j = tid; j < p.q_rank; j += 256) qo[j] = from_f32<T>(to_f32(row[p.q_off + j]) * inv * to_f32(w[j]));
    }
    if (p.kv_rank <= 0) return;
    // ---- the key/value latent and the shared key part
    __syncthreads();
    float ss = 0.f;
    for (int j = tid; j < p.kv_rank; j += 256) {
        float v = to_f32(row[p.kv_off + j]);
        ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)p.kv_rank + p.eps);
    const int width = p.kv_rank + p.rope_dim;
    T* dense = (T*)p.kv_out + (size_t)t * width;
    T* paged = nullptr;
    if (p.append) {
        const int s = p.tok_seq[t];
        const int last = p.seq_len_before[s] + (p.seq_start[s + 1] - p.seq_start[s]) - 1;
        if (paged_survives(pos / LLB_PAGE, last / LLB_PAGE, p.ring, p.pinned))
            paged = (T*)p.pool + paged_row(p.page_table + (size_t)s * p.table_stride, p.ring, pos, 0, 1, width, p.pinned);
    }
    const TW* w = (const TW*)p.wkv;
    for (int j = tid; j < p.kv_rank; j += 256) {
        T v = from_f32<T>(to_f32(row[p.kv_off + j]) * inv * to_f32(w[j]));
        dense[j] = v;
        if (paged) paged[j] = v;
    }
    const int half = p.rot >> 1;
    for (int i = tid; i < half; i += 256) {
        const float c = p.cos_t[(size_t)pos * half + i], s = p.sin_t[(size_t)pos * half + i];
        const int ia = p.halves ? i : 2 * i, ib = p.halves ? i + half : 2 * i + 1;
        const float a = to_f32(row[p.kr_off + ia]), b = to_f32(row[p.kr_off + ib]);
        T x = from_f32<T>(a * c - b * s), y = from_f32<T>(b * c + a * s);
        dense[p.kv_rank + ia] = x;
        dense[p.kv_rank + ib] = y;
        if (paged) {
            paged[p.kv_rank + ia] = x;
            paged[p.kv_rank + ib] = y;
        }
    }
    for (int j = p.rot + tid; j < p.rope_dim; j += 256) {
        T v = row[p.kr_off + j];
        dense[p.kv_rank + j] = v;
        if (paged) paged[p.kv_rank + j] = v;
    }
}

LLB_API int llb_latent_prep(LatentPrepParams p, int dtype, int w_dtype, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            llb_launch(latent_prep_kernel<TT, TW>, dim3(T), dim3(256), 0, stream, p);
        });
    });
    return llb_status();
}

// rows [T, width] -> the tokens' rows of the paged cache (one key head of `width` elements, no values)
template <typename T>
__global__ void __launch_bounds__(128) latent_append_kernel(const T* __restrict__ rows, int width, const int* __restrict__ tok_pos,
                                                            const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                                            const int* __restrict__ seq_len_before, T* __restrict__ pool,
                                                            const int* __restrict__ page_table, int table_stride, int ring,
                                                            int pinned) {
    const int t = blockIdx.x;
    llb_grid_dependency_sync();
    const int pos = tok_pos[t], s = tok_seq[t];
    const int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
    if (!paged_survives(pos / LLB_PAGE, last / LLB_PAGE, ring, pinned)) return;
    T* dst = pool + paged_row(page_table + (size_t)s * table_stride, ring, pos, 0, 1, width, pinned);
    const T* src = rows + (size_t)t * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = src[j];
}

LLB_API int llb_latent_append(const void* rows, int dtype, int T, int width, const int* tok_pos, const int* tok_seq,
                              const int* seq_start, const int* seq_len_before, void* pool, const int* page_table,
                              int table_stride, int ring, int pinned, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT, {
        llb_launch(latent_append_kernel<TT>, dim3(T), dim3(128), 0, stream, (const TT*)rows, width, tok_pos, tok_seq,
                   seq_start, seq_len_before, (TT*)pool, page_table, table_stride, ring, pinned);
    });
    return llb_status();
}

// ------------------------------------------------------------------ per-head matrix product
constexpr int HM_TOK = 16;        // tokens of a block
constexpr int HM_COLS = 32;       // output columns of a block (one per lane)
constexpr int HM_WARPS = 4;       // warps of a block: each takes a quarter of the inputs
constexpr int HM_THREADS = HM_WARPS * 32;

struct HeadMatmulParams {
    const void* x;            // [T, x_stride]: head h's input at h * x_head
    int x_stride, x_head;
    const void* m;            // [H, n_in, n_out]
    void* y;                  // [T, y_stride]: head h's output at h * y_head
    int y_stride, y_head;
    int T, H, n_in, n_out;
    // tail: the `tail` elements after a head's n_in inputs go to y after its n_out outputs, the first `rot` of them
    // rotated in pairs (2i, 2i+1) by the token's position
    int tail, rot;
    const float* cos_t;
    const float* sin_t;
    int table_rows;
    const int* tok_pos;
    // factor: y[t, h, :] *= sigmoid(gate[t * gate_stride + h])
    const void* gate;
    int gate_stride;
    int* err;
    int halves;               // rotated pairs are (i, i + rot / 2) instead of (2i, 2i + 1)
    int gate_elems;           // the gate has a value per output element (at h * n_out + column) instead of one per head
};

template <typename T>
__global__ void __launch_bounds__(HM_THREADS) head_matmul_kernel(HeadMatmulParams p) {
    extern __shared__ float xs[];                     // [HM_TOK][n_in], then the warps' partial sums [HM_WARPS][HM_TOK][HM_COLS]
    float* part = xs + HM_TOK * p.n_in;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, h = blockIdx.y;
    const int t0 = blockIdx.x * HM_TOK, nt = min(HM_TOK, p.T - t0);
    const int col = blockIdx.z * HM_COLS + lane;
    const T* mh = (const T*)p.m + (size_t)h * p.n_in * p.n_out + min(col, p.n_out - 1);
    // the warp's share of the inputs; its first weights are fetched before the kernel ahead has finished
    const int per = (p.n_in + HM_WARPS - 1) / HM_WARPS, d0 = warp * per, d1 = min(p.n_in, d0 + per);
    llb_grid_dependency_sync();
    const T* xb = (const T*)p.x;
    // the tile's inputs: four loads a thread are requested before the first is stored
    for (int i0 = tid; i0 < HM_TOK * p.n_in; i0 += 4 * HM_THREADS) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * HM_THREADS, t = i / p.n_in, d = i - t * p.n_in;
            v[u] = (i < HM_TOK * p.n_in && t < nt) ? to_f32(xb[(size_t)(t0 + t) * p.x_stride + h * p.x_head + d]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * HM_THREADS;
            if (i < HM_TOK * p.n_in) xs[i] = v[u];
        }
    }
    __syncthreads();
    T* yb = (T*)p.y;
    if (p.n_out > 0) {
        float acc[HM_TOK];
#pragma unroll
        for (int t = 0; t < HM_TOK; ++t) acc[t] = 0.f;
        int d = d0;
        for (; d + 8 <= d1; d += 8) {                 // eight weights in flight
            float w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = to_f32(mh[(size_t)(d + e) * p.n_out]);
#pragma unroll
            for (int t = 0; t < HM_TOK; ++t) {
                const float* x = xs + t * p.n_in + d;
                float a = acc[t];
#pragma unroll
                for (int e = 0; e < 8; ++e) a = fmaf(x[e], w[e], a);
                acc[t] = a;
            }
        }
        for (; d < d1; ++d) {
            const float w = to_f32(mh[(size_t)d * p.n_out]);
#pragma unroll
            for (int t = 0; t < HM_TOK; ++t) acc[t] = fmaf(xs[t * p.n_in + d], w, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < HM_TOK; ++t) part[(warp * HM_TOK + t) * HM_COLS + lane] = acc[t];
        __syncthreads();
        // warp w finishes the tokens w, w + 4, ...: the four partial sums in a fixed order
        for (int t = warp; t < nt; t += HM_WARPS) {
            float v = (part[t * HM_COLS + lane] + part[(HM_TOK + t) * HM_COLS + lane]) +
                      (part[(2 * HM_TOK + t) * HM_COLS + lane] + part[(3 * HM_TOK + t) * HM_COLS + lane]);
            if (p.gate) {
                float g = to_f32(((const T*)p.gate)[(size_t)(t0 + t) * p.gate_stride + (p.gate_elems ? h * p.n_out + min(col, p.n_out - 1) : h)]);
                v *= 1.0f / (1.0f + expf(-g));
            }
            if (col < p.n_out) yb[(size_t)(t0 + t) * p.y_stride + h * p.y_head + col] = from_f32<T>(v);
        }
    }
    if (blockIdx.z == 0 && p.tail > 0) {
        const int half = p.rot >> 1;
        for (int i = tid; i < nt * half; i += HM_THREADS) {
            int t = i / half, j = i - t * half;
            int pos = p.tok_pos[t0 + t];
            if (pos < 0 || pos >= p.table_rows) {
                atomicExch(p.err, 2);
                continue;
            }
            const float c = p.cos_t[(size_t)pos * half + j], s = p.sin_t[(size_t)pos * half + j];
            const T* src = xb + (size_t)(t0 + t) * p.x_stride + h * p.x_head + p.n_in;
            T* dst = yb + (size_t)(t0 + t) * p.y_stride + h * p.y_head + p.n_out;
            const int ia = p.halves ? j : 2 * j, ib = p.halves ? j + half : 2 * j + 1;
            const float a = to_f32(src[ia]), b = to_f32(src[ib]);
            dst[ia] = from_f32<T>(a * c - b * s);
            dst[ib] = from_f32<T>(b * c + a * s);
        }
        const int rest = p.tail - p.rot;
        for (int i = tid; i < nt * rest; i += HM_THREADS) {
            int t = i / rest, j = p.rot + i - t * rest;
            yb[(size_t)(t0 + t) * p.y_stride + h * p.y_head + p.n_out + j] =
                xb[(size_t)(t0 + t) * p.x_stride + h * p.x_head + p.n_in + j];
        }
    }
}

LLB_API int llb_head_matmul(HeadMatmulParams p, int dtype, cudaStream_t stream) {
    if (p.T == 0 || p.H == 0) return 0;
    size_t smem = (size_t)(HM_TOK * p.n_in + HM_WARPS * HM_TOK * HM_COLS) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid((p.T + HM_TOK - 1) / HM_TOK, p.H, p.n_out > 0 ? (p.n_out + HM_COLS - 1) / HM_COLS : 1);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, TT, {
        auto k = head_matmul_kernel<TT>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        llb_launch(k, grid, dim3(HM_THREADS), smem, stream, p);
    });
    return llb_status();
}

// ------------------------------------------------------------------ rotation and gate alone, in place
// x [T, stride]: H heads of `head` elements; the pairs (2i, 2i+1), i < rot / 2, of the elements from `off` on are rotated.
template <typename T>
__global__ void __launch_bounds__(128) rope_pairs_kernel(T* __restrict__ x, int stride, int H, int head, int off, int rot,
                                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                         int table_rows, const int* __restrict__ tok_pos, int* err, int halves) {
    const int t = blockIdx.x, pos = tok_pos[t], half = rot >> 1;
    if (pos < 0 || pos >= table_rows) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    llb_grid_dependency_sync();
    T* row = x + (size_t)t * stride;
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
        T* ea = row + h * head + off + (halves ? j : 2 * j);
        T* eb = row + h * head + off + (halves ? j + half : 2 * j + 1);
        const float a = to_f32(*ea), b = to_f32(*eb);
        *ea = from_f32<T>(a * c - b * s);
        *eb = from_f32<T>(b * c + a * s);
    }
}

LLB_API int llb_rope_pairs(void* x, int dtype, int T, int stride, int H, int head, int off, int rot, const float* cos_t,
                           const float* sin_t, int table_rows, const int* tok_pos, int* err, int halves, cudaStream_t stream) {
    if (T == 0 || rot <= 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT, {
        llb_launch(rope_pairs_kernel<TT>, dim3(T), dim3(128), 0, stream, (TT*)x, stride, H, head, off, rot, cos_t, sin_t,
                   table_rows, tok_pos, err, halves);
    });
    return llb_status();
}

// x[t, h, :] *= sigmoid(gate[t * gate_stride + h]) for x [T, H * width] (contiguous)
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, int gate_stride, int H, int width, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t th = i / width, t = th / H;
    int h = (int)(th - t * H);
    float g = to_f32(gate[t * gate_stride + h]);
    x[i] = from_f32<T>(to_f32(x[i]) / (1.0f + expf(-g)));
}

// bfloat16, head width a multiple of 8, 16-byte aligned: a thread takes eight neighbouring elements of one head
__global__ void head_gate_vec_kernel(bf16* __restrict__ x, const bf16* __restrict__ gate, int gate_stride, int H, int width8, size_t n8) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    size_t th = i / width8, t = th / H;
    int h = (int)(th - t * H);
    const float f = 1.0f / (1.0f + expf(-__bfloat162float(gate[t * gate_stride + h])));
    uint4 v = reinterpret_cast<uint4*>(x)[i];
    bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
    for (int k = 0; k < 8; ++k) e[k] = __float2bfloat16_rn(__bfloat162float(e[k]) * f);
    reinterpret_cast<uint4*>(x)[i] = v;
}

// bfloat16, one gate an element (heads of width 1), rows of a multiple of 8 elements, both 16-byte aligned: a thread takes
// eight neighbouring elements and their eight gates
__global__ void elem_gate_vec_kernel(bf16* __restrict__ x, const bf16* __restrict__ gate, int gate_stride, int H8, size_t n8) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const size_t t = i / H8;
    const int c = (int)(i - t * H8);
    uint4 v = reinterpret_cast<uint4*>(x)[i];
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + t * gate_stride + (size_t)c * 8);
    bf16* e = reinterpret_cast<bf16*>(&v);
    const bf16* g = reinterpret_cast<const bf16*>(&gv);
#pragma unroll
    for (int k = 0; k < 8; ++k) e[k] = __float2bfloat16_rn(__bfloat162float(e[k]) / (1.0f + expf(-__bfloat162float(g[k]))));
    reinterpret_cast<uint4*>(x)[i] = v;
}

LLB_API int llb_head_gate(void* x, const void* gate, int gate_stride, int dtype, int T, int H, int width, cudaStream_t stream) {
    size_t n = (size_t)T * H * width;
    if (n == 0) return 0;
    if (dtype == LLB_BF16 && width == 1 && H % 8 == 0 && gate_stride % 8 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)gate & 15)) {
        llb_launch(elem_gate_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (bf16*)x, (const bf16*)gate,
                   gate_stride, H / 8, n / 8);
        return llb_status();
    }
    if (dtype == LLB_BF16 && width % 8 == 0 && !((uintptr_t)x & 15)) {
        llb_launch(head_gate_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (bf16*)x, (const bf16*)gate,
                   gate_stride, H, width / 8, n / 8);
        return llb_status();
    }
    LLB_DISPATCH_DTYPE(dtype, TT, {
        llb_launch(head_gate_kernel<TT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (TT*)x, (const TT*)gate,
                   gate_stride, H, width, n);
    });
    return llb_status();
}
