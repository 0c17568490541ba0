// What happens to the heads of a packed projection between the matrix product and the attention kernel, and after it,
// for mixers whose heads are normed, rotated, pooled or combined:
//
//   head_prep     every query row and every key row of d elements: RMS norm over the row with a weight shared by all
//                 rows of its kind (optional), rotation of the row's first `rot` elements by the token's position
//                 (pairs (i, i + rot/2) or (2i, 2i+1)), in place and in float32 with one rounding; then (optionally) the
//                 keys and values go to the token's row of the paged cache.  A key/value head's cache row may hold
//                 several key rows side by side (a head with more than one score map).
//   pool_append   mean key and mean value of every block of P consecutive positions that the step completes, written to
//                 row `block` of a second paged cache (one row per block, every block kept).  Positions of the step are
//                 read from the projections, earlier ones from the token cache; sums in float32.
//   diff_combine  two attention results per head over the same values, a1 and a2: o = a1 - lambda a2, divided by its root
//                 mean square over the head's elements, times a constant.
#include "common.cuh"

struct HeadPrepParams {
    void* proj;               // [T, row_stride]: n_q query rows of d, then n_k key rows of d, then kv_heads value rows of dv
    int row_stride;
    int n_q, n_k, d;
    int kv_heads, dv;         // heads of the cache: a cache key row holds n_k / kv_heads key rows
    const float* q_weight;    // [d] or null: no norm of the query rows
    const float* k_weight;    // [d] or null
    float eps;
    int rot, layout;          // layout 0: pairs (i, i + rot/2); 1: pairs (2i, 2i + 1)
    const float* cos_t;       // [table_rows, rot / 2]
    const float* sin_t;
    int table_rows;
    const int* tok_pos;
    int append;
    const int* tok_seq;
    const int* seq_start;
    const int* seq_len_before;
    void* kpool;
    void* vpool;
    const int* page_table;
    int table_stride, ring, pinned;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(128) head_prep_kernel(HeadPrepParams p) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    llb_grid_dependency_sync();
    const int pos = p.tok_pos[t], half = p.rot >> 1, d = p.d;
    if (half > 0 && (pos < 0 || pos >= p.table_rows)) {
        if (threadIdx.x == 0) atomicExch(p.err, 2);
        return;
    }
    T* row = (T*)p.proj + (size_t)t * p.row_stride;
    const float* cs = p.cos_t + (size_t)pos * half;
    const float* sn = p.sin_t + (size_t)pos * half;
    for (int r = warp; r < p.n_q + p.n_k; r += 4) {
        T* x = row + (size_t)r * d;
        const float* w = r < p.n_q ? p.q_weight : p.k_weight;
        float inv = 1.f;
        if (w) {
            float ss = 0.f;
            for (int i = lane; i < d; i += 32) {
                const float v = to_f32(x[i]);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)d + p.eps);
        } else if (half == 0) {
            continue;
        }
        // (a lane reads and writes both elements of its pairs, and the sum above is complete: in place is safe)
        for (int j = lane; j < half; j += 32) {
            const int ia = p.layout ? 2 * j : j, ib = p.layout ? 2 * j + 1 : j + half;
            float a = to_f32(x[ia]), b = to_f32(x[ib]);
            if (w) {
                a = a * inv * w[ia];
                b = b * inv * w[ib];
            }
            const float c = cs[j], s = sn[j];
            x[ia] = from_f32<T>(a * c - b * s);
            x[ib] = from_f32<T>(b * c + a * s);
        }
        if (w)
            for (int i = p.rot + lane; i < d; i += 32) x[i] = from_f32<T>(to_f32(x[i]) * inv * w[i]);
    }
    if (!p.append) return;
    const int s = p.tok_seq[t];
    const int last = p.seq_len_before[s] + (p.seq_start[s + 1] - p.seq_start[s]) - 1;
    if (!paged_survives(pos / LLB_PAGE, last / LLB_PAGE, p.ring, p.pinned)) return;
    __syncthreads();
    const int* table = p.page_table + (size_t)s * p.table_stride;
    const int dkc = (p.n_k / p.kv_heads) * d;
    const T* k = row + (size_t)p.n_q * d;
    const T* v = k + (size_t)p.n_k * d;
    T* kpool = (T*)p.kpool;
    T* vpool = (T*)p.vpool;
    for (int i = threadIdx.x; i < p.kv_heads * dkc; i += blockDim.x) {
        const int h = i / dkc, j = i - h * dkc;
        kpool[paged_row(table, p.ring, pos, h, p.kv_heads, dkc, p.pinned) + j] = k[i];
    }
    for (int i = threadIdx.x; i < p.kv_heads * p.dv; i += blockDim.x) {
        const int h = i / p.dv, j = i - h * p.dv;
        vpool[paged_row(table, p.ring, pos, h, p.kv_heads, p.dv, p.pinned) + j] = v[i];
    }
}

LLB_API int llb_head_prep(HeadPrepParams p, int dtype, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    if (p.rot % 2 || p.rot < 0 || p.rot > p.d || p.d <= 0 || p.n_q < 0 || p.n_k < 0) return (int)cudaErrorInvalidValue;
    if (p.append && (p.kv_heads <= 0 || p.n_k % p.kv_heads)) return (int)cudaErrorInvalidValue;
    if (p.rot == 0 && !p.q_weight && !p.k_weight && !p.append) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT, llb_launch(head_prep_kernel<TT>, dim3(T), dim3(128), 0, stream, p));
    return llb_status();
}

// ------------------------------------------------------------------ pooled blocks
struct PoolAppendParams {
    const void* k_new;        // the step's keys as the cache will hold them: [T, row_stride] at the first key column
    const void* v_new;        // the same buffer at its first value column
    int row_stride;
    int kv_heads, dk, dv;     // dk: elements of a cache key row
    int pool;                 // positions of a block
    const void* kpool;        // the token cache (positions before the step)
    const void* vpool;
    const int* page_table;
    int table_stride, ring, pinned;
    void* pk;                 // the cache of blocks: row b of a sequence is block b
    void* pv;
    const int* ptable;
    int ptable_stride;
    const int* seq_start;
    const int* seq_len_before;
};

template <typename T>
__global__ void __launch_bounds__(128) pool_append_kernel(PoolAppendParams p) {
    extern __shared__ __align__(16) unsigned char pool_smem[];
    const T** krow = reinterpret_cast<const T**>(pool_smem);          // where each position's key row of this head lies
    const T** vrow = krow + p.pool;
    const int b = blockIdx.y, h = blockIdx.z;                  // a block per (block of positions, sequence, head)
    llb_grid_dependency_sync();
    const int tok0 = p.seq_start[b], n_new = p.seq_start[b + 1] - tok0, before = p.seq_len_before[b];
    const int blk = before / p.pool + blockIdx.x;              // blocks before it were complete before the step
    if (blk >= (before + n_new) / p.pool) return;
    const int* table = p.page_table + (size_t)b * p.table_stride;
    const int* ptable = p.ptable + (size_t)b * p.ptable_stride;
    for (int u = threadIdx.x; u < p.pool; u += blockDim.x) {
        const int pos = blk * p.pool + u;
        if (pos >= before) {
            const size_t at = (size_t)(tok0 + pos - before) * p.row_stride;
            krow[u] = (const T*)p.k_new + at + h * p.dk;
            vrow[u] = (const T*)p.v_new + at + h * p.dv;
        } else {
            krow[u] = (const T*)p.kpool + paged_row(table, p.ring, pos, h, p.kv_heads, p.dk, p.pinned);
            vrow[u] = (const T*)p.vpool + paged_row(table, p.ring, pos, h, p.kv_heads, p.dv, p.pinned);
        }
    }
    __syncthreads();
    const float inv = 1.0f / (float)p.pool;
    for (int j = threadIdx.x; j < p.dk + p.dv; j += blockDim.x) {
        const bool is_k = j < p.dk;
        const int e = is_k ? j : j - p.dk, w = is_k ? p.dk : p.dv;
        const T** rows = is_k ? krow : vrow;
        float acc = 0.f;
        int u = 0;
        for (; u + 8 <= p.pool; u += 8) {                      // eight loads in flight; the sum keeps the positions' order
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = to_f32(rows[u + i][e]);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc += x[i];
        }
        for (; u < p.pool; ++u) acc += to_f32(rows[u][e]);
        T* dst = (T*)(is_k ? p.pk : p.pv);
        dst[paged_row(ptable, p.ptable_stride, blk, h, p.kv_heads, w, 0) + e] = from_f32<T>(acc * inv);
    }
}

LLB_API int llb_pool_append(PoolAppendParams p, int dtype, int B, int max_new, cudaStream_t stream) {
    if (B == 0 || max_new == 0) return 0;
    if (p.pool <= 0 || p.kv_heads <= 0) return (int)cudaErrorInvalidValue;
    dim3 grid((max_new + p.pool - 1) / p.pool, B, p.kv_heads);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)p.pool * 2 * sizeof(void*);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, TT, llb_launch(pool_append_kernel<TT>, grid, dim3(128), smem, stream, p));
    return llb_status();
}

// ------------------------------------------------------------------ difference of two score maps' results
// a [T, 2 H dv] float32 holds, for key/value group g (r = H / G query heads each), first the r heads' results of map 1 and
// then those of map 2: head (g, m, j) at ((g * 2 + m) * r + j) * dv.  out [T, H dv]: head g * r + j.
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ a, T* __restrict__ out, int rows, int H, int r, int dv, float lambda, float eps,
                    float mult) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);       // (token, head)
    llb_grid_dependency_sync();
    if (row >= rows) return;
    const int t = row / H, h = row - t * H, g = h / r, j = h - g * r;
    const float* a1 = a + ((size_t)t * 2 * H + (size_t)(g * 2) * r + j) * dv;
    const float* a2 = a1 + (size_t)r * dv;
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) {
        const float o = a1[e] - lambda * a2[e];
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float inv = mult / sqrtf(ss / (float)dv + eps);
    for (int e = lane; e < dv; e += 32) out[(size_t)row * dv + e] = from_f32<T>((a1[e] - lambda * a2[e]) * inv);
}

LLB_API int llb_diff_combine(const float* a, void* out, int dtype, int T, int H, int r, int dv, float lambda, float eps, float mult,
                             cudaStream_t stream) {
    const int rows = T * H;
    if (rows == 0) return 0;
    if (r <= 0 || H % r) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, TT, llb_launch(diff_combine_kernel<TT>, dim3((rows + 3) / 4), dim3(128), 0, stream, a, (TT*)out, rows,
                                              H, r, dv, lambda, eps, mult));
    return llb_status();
}
