// Row-wise and element-wise kernels of the decoder: embedding gather, residual add fused with
// RMSNorm, half-split rotary encoding fused with the append to the paged cache, SwiGLU.
//
// Conventions: the residual stream is float32 in both precisions; activations that feed a
// matrix product have the model's activation dtype; sums of squares, the reciprocal root, the
// rotation and the residual sum are float32.  Formulas follow xsmccc/llaisys' CPU operators
// (src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34, src/ops/rope/cpu/rope_cpu.cpp:16-46,
// src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21, src/ops/embedding/cpu/embedding_cpu.cpp:16-22).
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int H, int V, int* err) {
    llb_grid_dependency_sync();
    int t = blockIdx.x;
    int id = ids[t];
    bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicExch(err, 1);
    const TW* row = table + (size_t)(ok ? id : 0) * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x)
        out[(size_t)t * H + j] = ok ? to_f32(row[j]) : 0.f;
}

LLB_API int llb_embedding(float* out, const void* table, int table_dtype, const int* ids, int T,
                          int H, int V, int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_DISPATCH_DTYPE(table_dtype, TW,
        llb_launch(embedding_kernel<TW>, dim3(T), dim3(256), 0, stream, out, (const TW*)table, ids, H, V, err));
    return llb_status();
}

// ------------------------------------------------------------------ token ids that stay on the device
// dst[i] = src[idx[i]] and dst[idx[i]] = src[i]: the last sampled token of every cache slot is kept in a table
// on the device, written after sampling and read by the next step, so that the next step can be launched
// before the host has seen the tokens.
__global__ void gather_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ idx, int n) {
    llb_grid_dependency_sync();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[idx[i]];
}
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx, const int* __restrict__ src, int n) {
    llb_grid_dependency_sync();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[idx[i]] = src[i];
}
LLB_API int llb_gather_i32(int* dst, const int* src, const int* idx, int n, cudaStream_t stream) {
    if (n == 0) return 0;
    llb_launch(gather_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, dst, src, idx, n);
    return llb_status();
}
LLB_API int llb_scatter_i32(int* dst, const int* idx, const int* src, int n, cudaStream_t stream) {
    if (n == 0) return 0;
    llb_launch(scatter_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, dst, idx, src, n);
    return llb_status();
}

// ------------------------------------------------------------------ residual add + RMSNorm
// Row r of the output is norm(residual[src] + sum_p delta[p][src]) with src = rows ? rows[r] : r.
// When write_back is set the summed row replaces residual[src] (never together with `rows`).
template <typename TD, typename TW, typename TO, int PER>     // PER > 0: H <= PER * 256 and the row lives in registers
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_part, size_t part_stride,
                   const TW* __restrict__ weight, TO* __restrict__ out, const int* __restrict__ rows, int H,
                   float eps, int write_back) {
    extern __shared__ float rowbuf[];          // H floats when PER == 0
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x;
    float x[PER > 0 ? PER : 1], w[PER > 0 ? PER : 1];
    if (PER > 0) {                             // the norm weight depends on no earlier kernel: fetch it first
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int j = tid + i * 256;
            w[i] = (j < H && out) ? to_f32(weight[j]) : 0.f;
        }
    }
    llb_grid_dependency_sync();
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * H;
    float ss = 0.f;
    if (PER > 0) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int j = tid + i * 256;
            x[i] = j < H ? res[j] : 0.f;
        }
        if (delta) {
            // the partial sums are added to one another first, then to the residual, as in the general path
            float d[PER > 0 ? PER : 1];
#pragma unroll
            for (int i = 0; i < PER; ++i) d[i] = 0.f;
            for (int p = 0; p < n_part; ++p) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    int j = tid + i * 256;
                    if (j < H) d[i] += to_f32(delta[p * part_stride + src * H + j]);
                }
            }
#pragma unroll
            for (int i = 0; i < PER; ++i) x[i] += d[i];
            if (write_back) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    int j = tid + i * 256;
                    if (j < H) res[j] = x[i];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) ss += x[i] * x[i];
    } else {
        for (int j = tid; j < H; j += 256) {
            float v = res[j];
            if (delta) {
                float d = 0.f;
                for (int p = 0; p < n_part; ++p) d += to_f32(delta[p * part_stride + src * H + j]);
                v += d;
                if (write_back) res[j] = v;
            }
            rowbuf[j] = v;
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    const int lane = tid & 31, wp = tid >> 5;
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    if (!out) return;
    if (PER > 0) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int j = tid + i * 256;
            if (j < H) out[(size_t)r * H + j] = from_f32<TO>(x[i] * w[i] * inv);
        }
    } else {
        for (int j = tid; j < H; j += 256)
            out[(size_t)r * H + j] = from_f32<TO>(rowbuf[j] * to_f32(weight[j]) * inv);
    }
}

// The same for the common case of the bfloat16 path (bfloat16 delta, weight and output, a width that is a multiple
// of 8 up to 8192, 16-byte aligned rows): a thread owns groups of eight consecutive columns, so that every access is a
// 16-byte one (two for the float32 residual).  Sums are formed in the same order as above.
template <int GROUPS>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const bf16* __restrict__ delta, int n_part, size_t part_stride,
                       const bf16* __restrict__ weight, bf16* __restrict__ out, const int* __restrict__ rows, int H,
                       float eps, int write_back) {
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x, n_groups = H >> 3;
    uint4 w[GROUPS];
#pragma unroll
    for (int i = 0; i < GROUPS; ++i) {         // the norm weight depends on no earlier kernel: fetch it first
        const int gidx = tid + i * 256;
        w[i] = (gidx < n_groups && out) ? *reinterpret_cast<const uint4*>(weight + gidx * 8) : make_uint4(0, 0, 0, 0);
    }
    llb_grid_dependency_sync();
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * H;
    float x[GROUPS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < GROUPS; ++i) {
        const int gidx = tid + i * 256;
        if (gidx < n_groups) {
            const float4 a = *reinterpret_cast<const float4*>(res + gidx * 8), b = *reinterpret_cast<const float4*>(res + gidx * 8 + 4);
            x[i][0] = a.x; x[i][1] = a.y; x[i][2] = a.z; x[i][3] = a.w; x[i][4] = b.x; x[i][5] = b.y; x[i][6] = b.z; x[i][7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[i][e] = 0.f;
        }
    }
    if (delta) {
#pragma unroll
        for (int i = 0; i < GROUPS; ++i) {
            const int gidx = tid + i * 256;
            if (gidx >= n_groups) continue;
            float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < n_part; ++q) {
                const uint4 v = *reinterpret_cast<const uint4*>(delta + q * part_stride + src * H + gidx * 8);
                const bf16* e8 = reinterpret_cast<const bf16*>(&v);
#pragma unroll
                for (int e = 0; e < 8; ++e) d[e] += to_f32(e8[e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) x[i][e] += d[e];
            if (write_back) {
                *reinterpret_cast<float4*>(res + gidx * 8) = make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
                *reinterpret_cast<float4*>(res + gidx * 8 + 4) = make_float4(x[i][4], x[i][5], x[i][6], x[i][7]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < GROUPS; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[i][e] * x[i][e];
    ss = warp_sum(ss);
    const int lane = tid & 31, wp = tid >> 5;
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    if (!out) return;
#pragma unroll
    for (int i = 0; i < GROUPS; ++i) {
        const int gidx = tid + i * 256;
        if (gidx >= n_groups) continue;
        const bf16* w8 = reinterpret_cast<const bf16*>(&w[i]);
        uint4 o;
        bf16* o8 = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = from_f32<bf16>(x[i][e] * to_f32(w8[e]) * inv);
        *reinterpret_cast<uint4*>(out + (size_t)r * H + gidx * 8) = o;
    }
}

// The same once more for many rows (prefill): a warp owns a row, a lane G groups of eight columns 256 columns apart, so
// a row needs no barrier of the block and no shared memory, every load of a lane is in flight at once, and eight rows
// share a block (a block per row is 2,048 blocks of which a quarter run as a second, partial wave).
template <int G>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ residual, const bf16* __restrict__ delta, int n_part, size_t part_stride,
                        const bf16* __restrict__ weight, bf16* __restrict__ out, int R, int H, float eps) {
    const int lane = threadIdx.x & 31, r = blockIdx.x * 8 + (threadIdx.x >> 5);
    uint4 w[G];
#pragma unroll
    for (int i = 0; i < G; ++i) w[i] = *reinterpret_cast<const uint4*>(weight + (lane + i * 32) * 8);      // depends on no earlier kernel
    llb_grid_dependency_sync();
    if (r >= R) return;
    float* res = residual + (size_t)r * H;
    float x[G][8];
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int c = (lane + i * 32) * 8;
        const float4 a = *reinterpret_cast<const float4*>(res + c), b = *reinterpret_cast<const float4*>(res + c + 4);
        x[i][0] = a.x; x[i][1] = a.y; x[i][2] = a.z; x[i][3] = a.w; x[i][4] = b.x; x[i][5] = b.y; x[i][6] = b.z; x[i][7] = b.w;
    }
    if (delta) {
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const int c = (lane + i * 32) * 8;
            float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < n_part; ++q) {
                const uint4 v = *reinterpret_cast<const uint4*>(delta + q * part_stride + (size_t)r * H + c);
                const bf16* e8 = reinterpret_cast<const bf16*>(&v);
#pragma unroll
                for (int e = 0; e < 8; ++e) d[e] += to_f32(e8[e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) x[i][e] += d[e];
            *reinterpret_cast<float4*>(res + c) = make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
            *reinterpret_cast<float4*>(res + c + 4) = make_float4(x[i][4], x[i][5], x[i][6], x[i][7]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < G; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[i][e] * x[i][e];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const bf16* w8 = reinterpret_cast<const bf16*>(&w[i]);
        uint4 o;
        bf16* o8 = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = from_f32<bf16>(x[i][e] * to_f32(w8[e]) * inv);
        *reinterpret_cast<uint4*>(out + (size_t)r * H + (lane + i * 32) * 8) = o;
    }
}

template <typename TD, typename TW>
static int add_rmsnorm_out(float* residual, const void* delta, int n_part, size_t part_stride,
                           const void* weight, void* out, int out_dtype, const int* rows, int R,
                           int H, float eps, int write_back, cudaStream_t stream) {
    size_t smem = (size_t)H * sizeof(float);
    LLB_DISPATCH_DTYPE(out_dtype, TO, {
        if (H <= 8 * 256) {
            llb_launch(add_rmsnorm_kernel<TD, TW, TO, 8>, dim3(R), dim3(256), 0, stream, residual, (const TD*)delta,
                       n_part, part_stride, (const TW*)weight, (TO*)out, rows, H, eps, write_back);
        } else {
            auto k = add_rmsnorm_kernel<TD, TW, TO, 0>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            llb_launch(k, dim3(R), dim3(256), smem, stream, residual, (const TD*)delta, n_part, part_stride,
                       (const TW*)weight, (TO*)out, rows, H, eps, write_back);
        }
    });
    return llb_status();
}

LLB_API int llb_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_part,
                            long long part_stride, const void* weight, int weight_dtype, void* out,
                            int out_dtype, const int* rows, int R, int H, float eps,
                            int write_back, cudaStream_t stream) {
    if (R == 0) return 0;
    if ((size_t)H * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (rows && write_back) return (int)cudaErrorInvalidValue;
    // the bfloat16 case with 16-byte accesses
    if ((!delta || delta_dtype == LLB_BF16) && weight_dtype == LLB_BF16 && (!out || out_dtype == LLB_BF16) && H % 8 == 0 &&
        H <= 8192 && part_stride % 8 == 0 &&
        !(((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15)) {
        // many whole rows, a width of G * 256 columns: a warp per row
        if (R >= 256 && !rows && out && write_back && H % 256 == 0 && H <= 4096) {
#define LLB_NW(G) case G: llb_launch(add_rmsnorm_warp_kernel<G>, dim3((R + 7) / 8), dim3(256), 0, stream, residual, (const bf16*)delta, \
                                     n_part, (size_t)part_stride, (const bf16*)weight, (bf16*)out, R, H, eps); return llb_status()
            switch (H / 256) {
                LLB_NW(1); LLB_NW(2); LLB_NW(3); LLB_NW(4); LLB_NW(5); LLB_NW(6); LLB_NW(7); LLB_NW(8);
                LLB_NW(9); LLB_NW(10); LLB_NW(11); LLB_NW(12); LLB_NW(13); LLB_NW(14); LLB_NW(15); LLB_NW(16);
            }
#undef LLB_NW
        }
#define LLB_NV(G) llb_launch(add_rmsnorm_vec_kernel<G>, dim3(R), dim3(256), 0, stream, residual, (const bf16*)delta, n_part, \
                             (size_t)part_stride, (const bf16*)weight, (bf16*)out, rows, H, eps, write_back)
        if (H <= 2048) LLB_NV(1);
        else if (H <= 4096) LLB_NV(2);
        else LLB_NV(4);
#undef LLB_NV
        return llb_status();
    }
    if (!delta) delta_dtype = LLB_F32;
    LLB_DISPATCH_DTYPE(delta_dtype, TD, {
        LLB_DISPATCH_DTYPE(weight_dtype, TW, {
            return add_rmsnorm_out<TD, TW>(residual, delta, n_part, (size_t)part_stride, weight, out,
                                           out_dtype, rows, R, H, eps, write_back, stream);
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ plain residual add
// residual[t] += sum_p delta[p][t]  (used where no norm follows).
template <typename TD>
__global__ void add_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_part,
                           size_t part_stride, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = 0.f;
    for (int p = 0; p < n_part; ++p) d += to_f32(delta[p * part_stride + i]);
    residual[i] += d;
}

LLB_API int llb_residual_add(float* residual, const void* delta, int delta_dtype, int n_part,
                             long long part_stride, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    LLB_DISPATCH_DTYPE(delta_dtype, TD,
        llb_launch(add_kernel<TD>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                   residual, (const TD*)delta, n_part, (size_t)part_stride, (size_t)n));
    return llb_status();
}

// ------------------------------------------------------------------ rotary + cache append
// qkv is the packed projection output [T, row_stride]: nh query heads, then nkvh key heads,
// then nkvh value heads, each of dh elements.  With ROPE the query and key heads are rotated in
// place (half-split pairs (j, j + dh/2), angle from the float32 cos/sin table built in double
// precision on the host).  With APPEND the (rotated) keys and the values of each token are
// written to the token's row of the paged cache.  A window layer keeps a ring of `ring` pages:
// tokens whose page would be overwritten within the same step are skipped.
template <typename T, bool ROPE, bool APPEND>
__global__ void rope_append_kernel(T* __restrict__ qkv, int row_stride, int nh, int nkvh, int dh,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   int table_rows, const int* __restrict__ tok_pos,
                                   const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                   const int* __restrict__ seq_len_before,
                                   T* __restrict__ kpool, T* __restrict__ vpool,
                                   const int* __restrict__ page_table, int table_stride, int ring,
                                   int* err) {
    llb_grid_dependency_sync();
    int t = blockIdx.x;
    int pos = tok_pos[t];
    T* row = qkv + (size_t)t * row_stride;
    int half = dh >> 1;
    const int* table = nullptr;
    bool store = false;
    if (APPEND) {
        int s = tok_seq[t];
        table = page_table + (size_t)s * table_stride;
        int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
        store = (pos / LLB_PAGE) + ring > (last / LLB_PAGE);
    }
    if (ROPE) {
        if (pos < 0 || pos >= table_rows) {
            if (threadIdx.x == 0) atomicExch(err, 2);
            return;
        }
        int n_rot = (nh + nkvh) * half;
        for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
            int h = i / half, j = i - h * half;
            float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
            T* x = row + h * dh;
            float a = to_f32(x[j]), b = to_f32(x[j + half]);
            T ya = from_f32<T>(a * c - b * s), yb = from_f32<T>(b * c + a * s);
            x[j] = ya;
            x[j + half] = yb;
            if (APPEND && store && h >= nh) {
                size_t o = paged_row(table, ring, pos, h - nh, nkvh, dh);
                kpool[o + j] = ya;
                kpool[o + j + half] = yb;
            }
        }
    } else if (APPEND && store) {
        for (int i = threadIdx.x; i < nkvh * dh; i += blockDim.x) {
            int h = i / dh, j = i - h * dh;
            kpool[paged_row(table, ring, pos, h, nkvh, dh) + j] = row[(nh + h) * dh + j];
        }
    }
    if (APPEND && store) {
        for (int i = threadIdx.x; i < nkvh * dh; i += blockDim.x) {
            int h = i / dh, j = i - h * dh;
            vpool[paged_row(table, ring, pos, h, nkvh, dh) + j] = row[(nh + nkvh + h) * dh + j];
        }
    }
}

// The same for bfloat16 rows whose head size is a multiple of 16 and whose rows start on 16-byte boundaries: a
// thread handles eight consecutive pairs (two 16-byte pieces of a head), so every access is a 16-byte one.
template <bool ROPE, bool APPEND>
__global__ void __launch_bounds__(128)
rope_append_vec_kernel(bf16* __restrict__ qkv, int row_stride, int nh, int nkvh, int dh,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_rows,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_len_before,
                       bf16* __restrict__ kpool, bf16* __restrict__ vpool, const int* __restrict__ page_table,
                       int table_stride, int ring, int* err) {
    // The step's index arrays reach the device by a copy that has ended before the step's first kernel starts, and the
    // rotation tables are older still, so they are read while the kernel before this one may still be running; its
    // output, the rows of qkv, only behind the dependency.
    const int t = blockIdx.x, pos = tok_pos[t], half = dh >> 1, vec_per_half = half >> 3;
    bf16* row = qkv + (size_t)t * row_stride;
    bool store = false;
    size_t page_base = 0;                     // element offset of the token's row of kv head 0 in the pools
    if (APPEND) {
        const int s = tok_seq[t];
        const int* table = page_table + (size_t)s * table_stride;
        const int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
        store = (pos / LLB_PAGE) + ring > (last / LLB_PAGE);
        if (store) page_base = paged_row(table, ring, pos, 0, nkvh, dh);
    }
    if (ROPE && (pos < 0 || pos >= table_rows)) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    const size_t head_step = (size_t)LLB_PAGE * dh;            // from one kv head's row to the next one's
    // the angles of this thread's first work item
    float4 pc0 = {}, pc1 = {}, ps0 = {}, ps1 = {};
    if (ROPE && (int)threadIdx.x < (nh + nkvh) * vec_per_half) {
        const int j = ((int)threadIdx.x % vec_per_half) * 8;
        pc0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j);
        pc1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j + 4);
        ps0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j);
        ps1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j + 4);
    }
    llb_grid_dependency_sync();
    // work items: (nh + nkvh) heads x vec_per_half pieces of rotation (or key copy), then nkvh x 2 vec_per_half of values
    const int n_rot = (nh + nkvh) * vec_per_half, n_val = APPEND && store ? nkvh * 2 * vec_per_half : 0;
    for (int i = threadIdx.x; i < n_rot + n_val; i += blockDim.x) {
        if (i < n_rot) {
            const int h = i / vec_per_half, j = (i - h * vec_per_half) * 8;
            if (!ROPE && !(APPEND && store && h >= nh)) continue;
            bf16* x = row + h * dh;
            uint4 lo = *reinterpret_cast<const uint4*>(x + j), hi = *reinterpret_cast<const uint4*>(x + j + half);
            if (ROPE) {
                float4 c0 = pc0, c1 = pc1, s0 = ps0, s1 = ps1;
                if (i != (int)threadIdx.x) {
                    c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j);
                    c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j + 4);
                    s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j);
                    s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j + 4);
                }
                const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                bf16* a = reinterpret_cast<bf16*>(&lo);
                bf16* b = reinterpret_cast<bf16*>(&hi);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float av = to_f32(a[e]), bv = to_f32(b[e]);
                    a[e] = from_f32<bf16>(av * c[e] - bv * sn[e]);
                    b[e] = from_f32<bf16>(bv * c[e] + av * sn[e]);
                }
                *reinterpret_cast<uint4*>(x + j) = lo;
                *reinterpret_cast<uint4*>(x + j + half) = hi;
            }
            if (APPEND && store && h >= nh) {
                const size_t o = page_base + (size_t)(h - nh) * head_step;
                *reinterpret_cast<uint4*>(kpool + o + j) = lo;
                *reinterpret_cast<uint4*>(kpool + o + j + half) = hi;
            }
        } else {
            const int v = i - n_rot, h = v / (2 * vec_per_half), j = (v - h * 2 * vec_per_half) * 8;
            *reinterpret_cast<uint4*>(vpool + page_base + (size_t)h * head_step + j) =
                *reinterpret_cast<const uint4*>(row + (nh + nkvh + h) * dh + j);
        }
    }
}

template <typename TT>
static void launch_rope_append(TT* qkv, int T, int row_stride, int nh, int nkvh, int dh, int do_rope,
                               const float* cos_t, const float* sin_t, int table_rows,
                               const int* tok_pos, int do_append, const int* tok_seq,
                               const int* seq_start, const int* seq_len_before, TT* kpool, TT* vpool,
                               const int* page_table, int table_stride, int ring, int* err,
                               cudaStream_t stream) {
#define LLB_RA(R, A)                                                                          \
    llb_launch(rope_append_kernel<TT, R, A>, dim3(T), dim3(128), 0, stream,                   \
        qkv, row_stride, nh, nkvh, dh, cos_t, sin_t, table_rows, tok_pos, tok_seq, seq_start, \
        seq_len_before, kpool, vpool, page_table, table_stride, ring, err)
    if (do_rope && do_append) LLB_RA(true, true);
    else if (do_rope) LLB_RA(true, false);
    else if (do_append) LLB_RA(false, true);
#undef LLB_RA
}

// bfloat16 with 16-byte pieces where sizes and addresses allow it
static bool rope_vec_ok(const void* qkv, int row_stride, int dh, const void* cos_t, const void* sin_t, const void* kpool,
                        const void* vpool) {
    return dh % 16 == 0 && row_stride % 8 == 0 &&
           !(((uintptr_t)qkv | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)kpool | (uintptr_t)vpool) & 15);
}
static void launch_rope_append_vec(bf16* qkv, int T, int row_stride, int nh, int nkvh, int dh, int do_rope,
                                   const float* cos_t, const float* sin_t, int table_rows, const int* tok_pos,
                                   int do_append, const int* tok_seq, const int* seq_start, const int* seq_len_before,
                                   bf16* kpool, bf16* vpool, const int* page_table, int table_stride, int ring, int* err,
                                   cudaStream_t stream) {
#define LLB_RAV(R, A)                                                                         \
    llb_launch(rope_append_vec_kernel<R, A>, dim3(T), dim3(128), 0, stream,                   \
        qkv, row_stride, nh, nkvh, dh, cos_t, sin_t, table_rows, tok_pos, tok_seq, seq_start, \
        seq_len_before, kpool, vpool, page_table, table_stride, ring, err)
    if (do_rope && do_append) LLB_RAV(true, true);
    else if (do_rope) LLB_RAV(true, false);
    else if (do_append) LLB_RAV(false, true);
#undef LLB_RAV
}

LLB_API int llb_rope_append(void* qkv, int dtype, int T, int row_stride, int nh, int nkvh, int dh,
                            int do_rope, const float* cos_t, const float* sin_t, int table_rows,
                            const int* tok_pos, int do_append, const int* tok_seq,
                            const int* seq_start, const int* seq_len_before, void* kpool,
                            void* vpool, const int* page_table, int table_stride, int ring,
                            int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    if (dh % 2) return (int)cudaErrorInvalidValue;
    if (dtype == LLB_BF16 && rope_vec_ok(qkv, row_stride, dh, cos_t, sin_t, kpool, vpool)) {
        launch_rope_append_vec((bf16*)qkv, T, row_stride, nh, nkvh, dh, do_rope, cos_t, sin_t, table_rows, tok_pos,
                               do_append, tok_seq, seq_start, seq_len_before, (bf16*)kpool, (bf16*)vpool, page_table,
                               table_stride, ring, err, stream);
        return llb_status();
    }
    LLB_DISPATCH_DTYPE(dtype, TT,
        launch_rope_append<TT>((TT*)qkv, T, row_stride, nh, nkvh, dh, do_rope, cos_t, sin_t,
                               table_rows, tok_pos, do_append, tok_seq, seq_start, seq_len_before,
                               (TT*)kpool, (TT*)vpool, page_table, table_stride, ring, err, stream));
    return llb_status();
}

// ------------------------------------------------------------------ SwiGLU
// gate_up is [T, 2I] with the gate columns first; out[t, i] = up * gate / (1 + exp(-gate)).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int I, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t t = i / I;
    int c = (int)(i - t * I);
    float g = to_f32(gate_up[t * 2 * I + c]);
    float u = to_f32(gate_up[t * 2 * I + I + c]);
    out[i] = from_f32<T>(u * (g / (1.0f + expf(-g))));
}

LLB_API int llb_swiglu(void* out, const void* gate_up, int dtype, int T, int I, cudaStream_t stream) {
    size_t n = (size_t)T * I;
    if (n == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT,
        llb_launch(swiglu_kernel<TT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (TT*)out, (const TT*)gate_up, I, n));
    return llb_status();
}

// ------------------------------------------------------------------ the same on dense operands
// out = up * gate / (1 + exp(-gate)) and c = a + b on dense tensors of one dtype: the operators
// swiglu and add of xsmccc/llaisys (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21, src/ops/add/cpu/add_cpu.cpp:8-16)
// as the op-level interface exposes them; float32 arithmetic, one rounding at the output.
template <typename T, bool SWIGLU>
__global__ void dense_binary_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float x = to_f32(a[i]), y = to_f32(b[i]);
    out[i] = from_f32<T>(SWIGLU ? y * (x / (1.0f + expf(-x))) : x + y);
}

// op 0: out = a + b;  op 1: out = b * a / (1 + exp(-a))  (a the gate, b the up projection)
LLB_API int llb_dense_binary(void* out, const void* a, const void* b, int dtype, long long n, int op, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (op != 0 && op != 1) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    LLB_DISPATCH_DTYPE(dtype, TT, {
        if (op == 0) llb_launch(dense_binary_kernel<TT, false>, dim3(blocks), dim3(256), 0, stream, (TT*)out, (const TT*)a, (const TT*)b, (size_t)n);
        else llb_launch(dense_binary_kernel<TT, true>, dim3(blocks), dim3(256), 0, stream, (TT*)out, (const TT*)a, (const TT*)b, (size_t)n);
    });
    return llb_status();
}

// ------------------------------------------------------------------ scaled embedding + hashed pair embedding
// out[t] = table[id_t] * scale + pair_table[r_t].  r_t is the hash (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets of
// the token and the one before it in its sequence; a sequence's first token (position 0) takes row `buckets`, the table's
// last.  The token before the first one of a step lives in `last` (int32 [slots, 2]: token, its position), which the
// block of a sequence's first token of the step reads and then overwrites with the step's last token of that sequence.
// A `last` entry that is not the position just before (a step that was run twice) sets err = 3.  pair_table null: no
// pair term and no state.
template <typename TW>
__global__ void __launch_bounds__(256)
embedding_pair_kernel(float* __restrict__ out, const TW* __restrict__ table, const TW* __restrict__ pair_table,
                      const int* __restrict__ ids, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                      const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int* __restrict__ last,
                      int H, int V, float scale, long long buckets, long long mul_prev, long long mul_cur, int* err) {
    __shared__ int prev_s;
    llb_grid_dependency_sync();
    const int t = blockIdx.x, id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicExch(err, 1);
    long long prow = -1;
    if (pair_table) {
        const int pos = tok_pos[t], s = tok_seq[t], start = seq_start[s];
        if (threadIdx.x == 0) {
            int prev = -1;
            if (t > start) prev = ids[t - 1];
            else {
                int* st = last + 2 * (size_t)seq_slot[s];
                if (pos > 0) {
                    prev = st[0];
                    if (st[1] != pos - 1) atomicExch(err, 3);
                }
                const int end = seq_start[s + 1] - 1;
                st[0] = ids[end];
                st[1] = pos + (end - start);
            }
            prev_s = prev;
        }
        __syncthreads();
        const int prev = prev_s;
        if (pos == 0) prow = buckets;
        else if (prev >= 0 && prev < V && ok) {
            long long h = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
            prow = h < 0 ? h + buckets : h;
        }
    }
    const TW* row = table + (size_t)(ok ? id : 0) * H;
    const TW* pr = prow >= 0 ? pair_table + (size_t)prow * H : nullptr;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = ok ? to_f32(row[j]) * scale : 0.f;
        if (pr) v += to_f32(pr[j]);
        out[(size_t)t * H + j] = v;
    }
}

LLB_API int llb_embedding_pair(float* out, const void* table, const void* pair_table, int table_dtype, const int* ids,
                               const int* tok_pos, const int* tok_seq, const int* seq_start, const int* seq_slot, int* last,
                               int T, int H, int V, float scale, long long buckets, long long mul_prev, long long mul_cur,
                               int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    if (pair_table && buckets <= 0) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(table_dtype, TW,
        llb_launch(embedding_pair_kernel<TW>, dim3(T), dim3(256), 0, stream, out, (const TW*)table, (const TW*)pair_table, ids,
                   tok_pos, tok_seq, seq_start, seq_slot, last, H, V, scale, buckets, mul_prev, mul_cur, err));
    return llb_status();
}

// ------------------------------------------------------------------ one root mean square, several weights
// out_i[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w_i for i < n (n = 1 or 2): the norms of the branches of a layer
// whose branches all read the same stream.  x is the float32 stream and is not written.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_multi_kernel(const float* __restrict__ x, const TW* __restrict__ w0, const TW* __restrict__ w1,
                     TO* __restrict__ out0, TO* __restrict__ out1, int H, float eps) {
    __shared__ float red[8];
    llb_grid_dependency_sync();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = x + (size_t)r * H;
    float ss = 0.f;
    for (int j = tid; j < H; j += 256) {
        float v = row[j];
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    for (int j = tid; j < H; j += 256) {
        const float v = row[j] * inv;
        out0[(size_t)r * H + j] = from_f32<TO>(v * to_f32(w0[j]));
        if (out1) out1[(size_t)r * H + j] = from_f32<TO>(v * to_f32(w1[j]));
    }
}

LLB_API int llb_rmsnorm_multi(const float* x, const void* w0, const void* w1, int w_dtype, void* out0, void* out1,
                              int out_dtype, int R, int H, float eps, cudaStream_t stream) {
    if (R == 0) return 0;
    LLB_DISPATCH_DTYPE(w_dtype, TW, {
        LLB_DISPATCH_DTYPE(out_dtype, TO, {
            llb_launch(rmsnorm_multi_kernel<TW, TO>, dim3(R), dim3(256), 0, stream, x, (const TW*)w0, (const TW*)w1,
                       (TO*)out0, (TO*)out1, H, eps);
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ rotation of a head's leading dimensions + cache append
// proj is a packed projection output [T, row_stride]: nh query heads of dk elements; then, when the layer projects keys
// and values of its own (nkvh > 0), nkvh key heads of dk and nkvh value heads of dv elements.  The first `rot` dimensions
// of every query and key head are rotated in pairs (j, j + rot/2) by the angle of cos_t/sin_t [rows, rot/2] at the
// token's position; the dimensions from `rot` on pass unchanged.  With APPEND the (rotated) keys and the values are
// written to the token's row of the paged cache (ring of `ring` pages behind `pinned` pages that are never overwritten).
template <typename T, bool APPEND>
__global__ void __launch_bounds__(128)
rope_lead_append_kernel(T* __restrict__ proj, int row_stride, int nh, int nkvh, int dk, int dv, int rot,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_rows,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_len_before,
                        T* __restrict__ kpool, T* __restrict__ vpool, const int* __restrict__ page_table,
                        int table_stride, int ring, int pinned, int* err) {
    const int t = blockIdx.x, pos = tok_pos[t], half = rot >> 1;
    const int* table = nullptr;
    bool store = false;
    if (APPEND) {
        const int s = tok_seq[t];
        table = page_table + (size_t)s * table_stride;
        const int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
        store = paged_survives(pos / LLB_PAGE, last / LLB_PAGE, ring, pinned);
    }
    if (half > 0 && (pos < 0 || pos >= table_rows)) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    llb_grid_dependency_sync();
    T* row = proj + (size_t)t * row_stride;
    for (int i = threadIdx.x; i < (nh + nkvh) * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
        T* x = row + h * dk;
        const float a = to_f32(x[j]), b = to_f32(x[j + half]);
        x[j] = from_f32<T>(a * c - b * s);
        x[j + half] = from_f32<T>(b * c + a * s);
    }
    if (APPEND && store) {
        __syncthreads();
        const T* k = row + nh * dk;
        const T* v = k + nkvh * dk;
        for (int i = threadIdx.x; i < nkvh * dk; i += blockDim.x) {
            const int h = i / dk, j = i - h * dk;
            kpool[paged_row(table, ring, pos, h, nkvh, dk, pinned) + j] = k[i];
        }
        for (int i = threadIdx.x; i < nkvh * dv; i += blockDim.x) {
            const int h = i / dv, j = i - h * dv;
            vpool[paged_row(table, ring, pos, h, nkvh, dv, pinned) + j] = v[i];
        }
    }
}

// The same for bfloat16 rows in 16-byte pieces: rot a multiple of 16, dk and dv multiples of 8, rows and pools on 16-byte
// boundaries.  A thread rotates eight consecutive pairs at a time and copies keys and values eight elements at a time.
template <bool APPEND>
__global__ void __launch_bounds__(128)
rope_lead_append_vec_kernel(bf16* __restrict__ proj, int row_stride, int nh, int nkvh, int dk, int dv, int rot,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_rows,
                            const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_len_before,
                            bf16* __restrict__ kpool, bf16* __restrict__ vpool, const int* __restrict__ page_table,
                            int table_stride, int ring, int pinned, int* err) {
    const int t = blockIdx.x, pos = tok_pos[t], half = rot >> 1, per_head = half >> 3;
    bool store = false;
    size_t k_base = 0, v_base = 0;            // element offsets of the token's row of kv head 0 in the pools
    if (APPEND) {
        const int s = tok_seq[t];
        const int* table = page_table + (size_t)s * table_stride;
        const int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
        store = paged_survives(pos / LLB_PAGE, last / LLB_PAGE, ring, pinned);
        if (store) {
            k_base = paged_row(table, ring, pos, 0, nkvh, dk, pinned);
            v_base = paged_row(table, ring, pos, 0, nkvh, dv, pinned);
        }
    }
    if (half > 0 && (pos < 0 || pos >= table_rows)) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    llb_grid_dependency_sync();
    bf16* row = proj + (size_t)t * row_stride;
    for (int i = threadIdx.x; i < (nh + nkvh) * per_head; i += blockDim.x) {
        const int h = i / per_head, j = (i - h * per_head) * 8;
        bf16* x = row + h * dk;
        uint4 lo = *reinterpret_cast<const uint4*>(x + j), hi = *reinterpret_cast<const uint4*>(x + j + half);
        const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j), c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j), s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j + 4);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        bf16* a = reinterpret_cast<bf16*>(&lo);
        bf16* b = reinterpret_cast<bf16*>(&hi);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float av = to_f32(a[e]), bv = to_f32(b[e]);
            a[e] = from_f32<bf16>(av * c[e] - bv * sn[e]);
            b[e] = from_f32<bf16>(bv * c[e] + av * sn[e]);
        }
        *reinterpret_cast<uint4*>(x + j) = lo;
        *reinterpret_cast<uint4*>(x + j + half) = hi;
    }
    if (APPEND && store) {
        __syncthreads();
        const bf16* k = row + nh * dk;
        const bf16* v = k + nkvh * dk;
        const int kc = dk >> 3, vc = dv >> 3;
        const size_t k_step = (size_t)LLB_PAGE * dk, v_step = (size_t)LLB_PAGE * dv;     // from one kv head's row to the next one's
        for (int i = threadIdx.x; i < nkvh * kc; i += blockDim.x) {
            const int h = i / kc, j = (i - h * kc) * 8;
            *reinterpret_cast<uint4*>(kpool + k_base + h * k_step + j) = *reinterpret_cast<const uint4*>(k + h * dk + j);
        }
        for (int i = threadIdx.x; i < nkvh * vc; i += blockDim.x) {
            const int h = i / vc, j = (i - h * vc) * 8;
            *reinterpret_cast<uint4*>(vpool + v_base + h * v_step + j) = *reinterpret_cast<const uint4*>(v + h * dv + j);
        }
    }
}

LLB_API int llb_rope_lead_append(void* proj, int dtype, int T, int row_stride, int nh, int nkvh, int dk, int dv, int rot,
                                 const float* cos_t, const float* sin_t, int table_rows, const int* tok_pos, int do_append,
                                 const int* tok_seq, const int* seq_start, const int* seq_len_before, void* kpool,
                                 void* vpool, const int* page_table, int table_stride, int ring, int pinned, int* err,
                                 cudaStream_t stream) {
    if (T == 0) return 0;
    if (rot % 2 || rot > dk || rot < 0) return (int)cudaErrorInvalidValue;
    if (rot == 0 && !do_append) return 0;
    if (dtype == LLB_BF16 && rot % 16 == 0 && dk % 8 == 0 && dv % 8 == 0 && row_stride % 8 == 0 &&
        !(((uintptr_t)proj | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)kpool | (uintptr_t)vpool) & 15)) {
#define LLB_RLAV(A)                                                                                                    \
    llb_launch(rope_lead_append_vec_kernel<A>, dim3(T), dim3(128), 0, stream, (bf16*)proj, row_stride, nh, nkvh, dk,   \
               dv, rot, cos_t, sin_t, table_rows, tok_pos, tok_seq, seq_start, seq_len_before, (bf16*)kpool,            \
               (bf16*)vpool, page_table, table_stride, ring, pinned, err)
        if (do_append) LLB_RLAV(true);
        else LLB_RLAV(false);
#undef LLB_RLAV
        return llb_status();
    }
#define LLB_RLA(A)                                                                                                     \
    llb_launch(rope_lead_append_kernel<TT, A>, dim3(T), dim3(128), 0, stream, (TT*)proj, row_stride, nh, nkvh, dk, dv,  \
               rot, cos_t, sin_t, table_rows, tok_pos, tok_seq, seq_start, seq_len_before, (TT*)kpool, (TT*)vpool,      \
               page_table, table_stride, ring, pinned, err)
    LLB_DISPATCH_DTYPE(dtype, TT, {
        if (do_append) LLB_RLA(true);
        else LLB_RLA(false);
    });
#undef LLB_RLA
    return llb_status();
}

// ------------------------------------------------------------------ squared ReLU
// x <- max(x, 0)^2 in place, float32 arithmetic, one rounding.
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ x, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = fmaxf(to_f32(x[i]), 0.f);
    x[i] = from_f32<T>(v * v);
}

// bfloat16, eight elements (16 bytes) per thread
__global__ void relu_squared_vec_kernel(bf16* __restrict__ x, size_t n8) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    uint4 v = reinterpret_cast<uint4*>(x)[i];
    bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float f = fmaxf(to_f32(e[k]), 0.f);
        e[k] = from_f32<bf16>(f * f);
    }
    reinterpret_cast<uint4*>(x)[i] = v;
}

LLB_API int llb_relu_squared(void* x, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == LLB_BF16 && n % 8 == 0 && !((uintptr_t)x & 15)) {
        const size_t n8 = (size_t)n / 8;
        llb_launch(relu_squared_vec_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, (bf16*)x, n8);
        return llb_status();
    }
    LLB_DISPATCH_DTYPE(dtype, TT,
        llb_launch(relu_squared_kernel<TT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (TT*)x, (size_t)n));
    return llb_status();
}

// ------------------------------------------------------------------ misc

// ------------------------------------------------------------------ a part's normed output into the stream (+ the next norm)
// residual[r] += mult * delta[r] / sqrt(mean(delta[r]^2) + eps) * (w_post + offset), all in float32; with `out` the same
// pass then normalises the new stream row with w_next: out[r] = residual[r] / sqrt(mean(residual[r]^2) + eps) *
// (w_next + offset), so that a layer whose parts sit between two norms needs one launch per part for its norms.
// Without delta only the second half runs (the plain norm of a row).  The row lives in shared memory (H floats).
template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(256)
scaled_norm_add_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const TW* __restrict__ w_post,
                       float mult, const TW* __restrict__ w_next, TO* __restrict__ out, int H, float eps, float offset) {
    extern __shared__ float rowbuf[];
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    llb_grid_dependency_sync();
    float* res = residual + (size_t)r * H;
    if (delta) {
        const TD* d = delta + (size_t)r * H;
        float ss = 0.f;
        for (int j = tid; j < H; j += 256) {
            float v = to_f32(d[j]);
            rowbuf[j] = v;
            ss += v * v;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[wp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot += red[i];
        const float inv = mult / sqrtf(tot / (float)H + eps);
        __syncthreads();
        for (int j = tid; j < H; j += 256) {
            float v = res[j] + rowbuf[j] * inv * (to_f32(w_post[j]) + offset);
            res[j] = v;
            rowbuf[j] = v;
        }
    } else {
        for (int j = tid; j < H; j += 256) rowbuf[j] = res[j];
    }
    if (!out) return;
    float ss = 0.f;
    for (int j = tid; j < H; j += 256) ss += rowbuf[j] * rowbuf[j];
    ss = warp_sum(ss);
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    for (int j = tid; j < H; j += 256)
        out[(size_t)r * H + j] = from_f32<TO>(rowbuf[j] * inv * (to_f32(w_next[j]) + offset));
}

LLB_API int llb_scaled_norm_add(float* residual, const void* delta, int delta_dtype, const void* w_post, float mult,
                                const void* w_next, int w_dtype, void* out, int out_dtype, int R, int H, float eps,
                                float offset, cudaStream_t stream) {
    if (R == 0) return 0;
    size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (!delta) delta_dtype = LLB_F32;
    if (!out) out_dtype = LLB_F32;
    LLB_DISPATCH_DTYPE(delta_dtype, TD, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            LLB_DISPATCH_DTYPE(out_dtype, TO, {
                auto k = scaled_norm_add_kernel<TD, TW, TO>;
                if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                llb_launch(k, dim3(R), dim3(256), smem, stream, residual, (const TD*)delta, (const TW*)w_post, mult,
                           (const TW*)w_next, (TO*)out, H, eps, offset);
            });
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ gated activation of a fused gate/up product
// gate_up is [T, 2I] with the gate columns first; out[t, i] = act(gate) * up, act: 0 silu, 1 relu, 2 gelu (tanh form);
// 3: the clamped form g' = min(gate, limit), u' = clamp(up, -limit, limit), out = g' sigmoid(alpha g') (u' + 1).
__device__ __forceinline__ float glu_clamped(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}
template <typename TI, typename TO>
__global__ void glu_kernel(TO* __restrict__ out, const TI* __restrict__ gate_up, int I, size_t n, int act, float limit, float alpha) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t t = i / I;
    int c = (int)(i - t * I);
    float g = to_f32(gate_up[t * 2 * I + c]);
    float u = to_f32(gate_up[t * 2 * I + I + c]);
    if (act == 3) {
        out[i] = from_f32<TO>(glu_clamped(g, u, limit, alpha));
        return;
    }
    float a;
    if (act == 1) a = fmaxf(g, 0.f);
    else if (act == 2) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else a = g / (1.0f + expf(-g));
    out[i] = from_f32<TO>(a * u);
}

// bfloat16 in and out, I a multiple of 8, 16-byte aligned: a thread takes eight neighbouring elements.
__device__ __forceinline__ float glu_act(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));
}
__global__ void glu_vec_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate_up, int I8, size_t n8, int act, float limit,
                               float alpha) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    size_t t = i / I8;
    int c = (int)(i - t * I8);
    const uint4 g = reinterpret_cast<const uint4*>(gate_up)[t * 2 * I8 + c];
    const uint4 u = reinterpret_cast<const uint4*>(gate_up)[t * 2 * I8 + I8 + c];
    const bf16* gv = reinterpret_cast<const bf16*>(&g);
    const bf16* uv = reinterpret_cast<const bf16*>(&u);
    uint4 o;
    bf16* ov = reinterpret_cast<bf16*>(&o);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float gf = __bfloat162float(gv[e]), uf = __bfloat162float(uv[e]);
        ov[e] = __float2bfloat16_rn(act == 3 ? glu_clamped(gf, uf, limit, alpha) : glu_act(gf, act) * uf);
    }
    reinterpret_cast<uint4*>(out)[i] = o;
}

LLB_API int llb_glu(void* out, int out_dtype, const void* gate_up, int in_dtype, int T, int I, int act, float limit, float alpha,
                    cudaStream_t stream) {
    size_t n = (size_t)T * I;
    if (n == 0) return 0;
    if (in_dtype == LLB_BF16 && out_dtype == LLB_BF16 && I % 8 == 0 && !(((uintptr_t)out | (uintptr_t)gate_up) & 15)) {
        llb_launch(glu_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (bf16*)out, (const bf16*)gate_up,
                   I / 8, n / 8, act, limit, alpha);
        return llb_status();
    }
    LLB_DISPATCH_DTYPE(in_dtype, TI, {
        LLB_DISPATCH_DTYPE(out_dtype, TO, {
            llb_launch(glu_kernel<TI, TO>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (TO*)out,
                       (const TI*)gate_up, I, n, act, limit, alpha);
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ stream update: scaled add, depth average, norm
// One pass over a row of the float32 stream for arrangements whose parts join the stream scaled and whose layers hand
// on a weighted sum of every earlier layer's result:
//   v      = cur[r] + delta_scale * sum_p delta[p][r]                (delta optional; written back to cur with write_back)
//   y      = mix ? sum_{j < n-1} mix[j] * X_j[r] + mix[n-1] * v : v   (X_0 = x0, X_j = planes + (j-1) * plane_stride for j >= 1;
//                                                                     the last of the n terms is the row just formed)
//   dst[r] = y                                                        (dst optional: the plane the next layer works on)
//   out[r] = y / sqrt(mean(y^2) + eps) * weight                       (out optional)
// With `rows` only the rows listed there are read, nothing is written back, and dst and out are [len(rows), H].
// Terms are added in ascending j, so a row's result does not depend on what else the step holds.
struct StreamUpdateParams {
    float* cur;               // [T, H] the row's current plane
    const void* delta;        // [n_part, T, H] or null
    int n_part;
    long long part_stride;
    float delta_scale;
    int write_back;
    const float* mix;         // [n] or null
    int n;                    // terms of the sum
    const float* x0;          // [T, H]
    const float* planes;      // [n - 2 planes of T * H ahead of cur's]
    long long plane_stride;
    float* dst;               // [R, H] or null
    const void* weight;       // [H]
    void* out;                // [R, H] or null
    const int* rows;          // [R] or null
    int H;
    float eps;
};

template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(256) stream_update_kernel(StreamUpdateParams p) {
    extern __shared__ float rowbuf[];
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5, H = p.H;
    llb_grid_dependency_sync();
    const size_t src = p.rows ? (size_t)p.rows[r] : (size_t)r;
    float* cur = p.cur + src * H;
    const TD* delta = (const TD*)p.delta;
    float ss = 0.f;
    for (int j = tid; j < H; j += 256) {
        float v = cur[j];
        if (delta) {
            float d = 0.f;
            for (int q = 0; q < p.n_part; ++q) d += to_f32(delta[(size_t)q * p.part_stride + src * H + j]);
            v = fmaf(p.delta_scale, d, v);
            if (p.write_back) cur[j] = v;
        }
        if (p.mix) {
            float acc = 0.f;
            if (p.n > 1) acc = p.mix[0] * p.x0[src * H + j];
            for (int k = 1; k + 1 < p.n; ++k) acc = fmaf(p.mix[k], p.planes[(size_t)(k - 1) * p.plane_stride + src * H + j], acc);
            v = fmaf(p.mix[p.n - 1], v, acc);
        }
        if (p.dst) p.dst[(size_t)r * H + j] = v;
        rowbuf[j] = v;
        ss += v * v;
    }
    if (!p.out) return;
    ss = warp_sum(ss);
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + p.eps);
    const TW* w = (const TW*)p.weight;
    TO* out = (TO*)p.out + (size_t)r * H;
    for (int j = tid; j < H; j += 256) out[j] = from_f32<TO>(rowbuf[j] * inv * to_f32(w[j]));
}

// The same with 16-byte accesses to the float32 planes (8-byte ones to bfloat16 operands): widths that are multiples
// of 4, aligned bases.  Sums are formed in the same order as above.
template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(256) stream_update_vec_kernel(StreamUpdateParams p) {
    extern __shared__ float rowbuf[];
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5, H = p.H, H4 = H >> 2;
    llb_grid_dependency_sync();
    const size_t src = p.rows ? (size_t)p.rows[r] : (size_t)r;
    float* cur = p.cur + src * H;
    const TD* delta = (const TD*)p.delta;
    float ss = 0.f;
    for (int g = tid; g < H4; g += 256) {
        const int j = g * 4;
        const float4 c4 = *reinterpret_cast<const float4*>(cur + j);
        float v[4] = {c4.x, c4.y, c4.z, c4.w};
        if (delta) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < p.n_part; ++q) {
                const TD* dp = delta + (size_t)q * p.part_stride + src * H + j;
                if (sizeof(TD) == 4) {
                    const float4 t = *reinterpret_cast<const float4*>(dp);
                    d[0] += t.x; d[1] += t.y; d[2] += t.z; d[3] += t.w;
                } else {
                    const uint2 t = *reinterpret_cast<const uint2*>(dp);
                    const TD* e = reinterpret_cast<const TD*>(&t);
#pragma unroll
                    for (int u = 0; u < 4; ++u) d[u] += to_f32(e[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = fmaf(p.delta_scale, d[u], v[u]);
            if (p.write_back) *reinterpret_cast<float4*>(cur + j) = make_float4(v[0], v[1], v[2], v[3]);
        }
        if (p.mix) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (p.n > 1) {
                const float a = p.mix[0];
                const float4 t = *reinterpret_cast<const float4*>(p.x0 + src * H + j);
                acc[0] = a * t.x; acc[1] = a * t.y; acc[2] = a * t.z; acc[3] = a * t.w;
            }
            for (int k = 1; k + 1 < p.n; ++k) {
                const float a = p.mix[k];
                const float4 t = *reinterpret_cast<const float4*>(p.planes + (size_t)(k - 1) * p.plane_stride + src * H + j);
                acc[0] = fmaf(a, t.x, acc[0]); acc[1] = fmaf(a, t.y, acc[1]); acc[2] = fmaf(a, t.z, acc[2]); acc[3] = fmaf(a, t.w, acc[3]);
            }
            const float a = p.mix[p.n - 1];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = fmaf(a, v[u], acc[u]);
        }
        if (p.dst) *reinterpret_cast<float4*>(p.dst + (size_t)r * H + j) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(rowbuf + j) = make_float4(v[0], v[1], v[2], v[3]);
        ss += (v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3]);
    }
    if (!p.out) return;
    ss = warp_sum(ss);
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + p.eps);
    const TW* w = (const TW*)p.weight;
    TO* out = (TO*)p.out + (size_t)r * H;
    for (int g = tid; g < H4; g += 256) {
        const int j = g * 4;
        const float4 x = *reinterpret_cast<const float4*>(rowbuf + j);
        const float y[4] = {x.x * inv * to_f32(w[j]), x.y * inv * to_f32(w[j + 1]), x.z * inv * to_f32(w[j + 2]), x.w * inv * to_f32(w[j + 3])};
        if (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(out + j) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
            uint2 o;
            TO* e = reinterpret_cast<TO*>(&o);
#pragma unroll
            for (int u = 0; u < 4; ++u) e[u] = from_f32<TO>(y[u]);
            *reinterpret_cast<uint2*>(out + j) = o;
        }
    }
}

LLB_API int llb_stream_update(StreamUpdateParams p, int delta_dtype, int w_dtype, int out_dtype, int R, cudaStream_t stream) {
    if (R == 0) return 0;
    const size_t smem = (size_t)p.H * sizeof(float);
    if (smem > 200 * 1024 || (p.mix && p.n < 1) || (p.rows && p.write_back)) return (int)cudaErrorInvalidValue;
    if (!p.delta) delta_dtype = LLB_F32;
    if (!p.out) { out_dtype = LLB_F32; w_dtype = LLB_F32; }
    const bool vec = p.H % 4 == 0 && p.part_stride % 4 == 0 && p.plane_stride % 4 == 0 &&
                     !(((uintptr_t)p.cur | (uintptr_t)p.delta | (uintptr_t)p.x0 | (uintptr_t)p.planes | (uintptr_t)p.dst | (uintptr_t)p.out) & 15);
    LLB_DISPATCH_DTYPE(delta_dtype, TD, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            LLB_DISPATCH_DTYPE(out_dtype, TO, {
                auto k = vec ? stream_update_vec_kernel<TD, TW, TO> : stream_update_kernel<TD, TW, TO>;
                if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                llb_launch(k, dim3(R), dim3(256), smem, stream, p);
            });
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ activation of rows, with a factor per row
// x[t, :cols] <- act(x[t, :cols]) * factor_t in place (row stride ldx), factor_t = scale * sigmoid(logit[t * ld_logit])
// (scale alone without logits); act 1: max(., 0)^2, 2: gelu (erf form), 3: gelu (tanh form).  float32 arithmetic, one rounding.
__device__ __forceinline__ float row_act(float v, int act) {
    if (act == 1) { v = fmaxf(v, 0.f); return v * v; }
    if (act == 2) return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
    if (act == 3) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

template <typename T>
__global__ void __launch_bounds__(256) act_rows_kernel(T* __restrict__ x, int ldx, int cols, int act, const float* __restrict__ logit,
                                                       int ld_logit, float scale) {
    const int t = blockIdx.x;
    llb_grid_dependency_sync();
    const float f = logit ? scale / (1.0f + expf(-logit[(size_t)t * ld_logit])) : scale;
    T* row = x + (size_t)t * ldx;
    constexpr int VEC = 16 / (int)sizeof(T);
    if (cols % VEC == 0 && ldx % VEC == 0 && !((uintptr_t)x & 15)) {
        for (int g = threadIdx.x; g < cols / VEC; g += 256) {
            uint4 v = reinterpret_cast<uint4*>(row)[g];
            T* e = reinterpret_cast<T*>(&v);
#pragma unroll
            for (int u = 0; u < VEC; ++u) e[u] = from_f32<T>(row_act(to_f32(e[u]), act) * f);
            reinterpret_cast<uint4*>(row)[g] = v;
        }
        return;
    }
    for (int j = threadIdx.x; j < cols; j += 256) row[j] = from_f32<T>(row_act(to_f32(row[j]), act) * f);
}

LLB_API int llb_act_rows(void* x, int dtype, int T, int ldx, int cols, int act, const float* logit, int ld_logit, float scale,
                         cudaStream_t stream) {
    if (T == 0 || cols == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT,
        llb_launch(act_rows_kernel<TT>, dim3(T), dim3(256), 0, stream, (TT*)x, ldx, cols, act, logit, ld_logit, scale));
    return llb_status();
}

LLB_API const char* llb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }
