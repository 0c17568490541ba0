// Passes over rows of the float32 residual stream for arrangements whose parts join the stream through a gate:
//
//   stream_join   v = x[r] + sigmoid(gate[r]) * delta[r] + rows_add[r] + vec_add        (each term optional; element by
//                 element; written back to x), then out[r] = v / sqrt(mean(v^2) + eps) * weight   (optional)
//   branch_mean   out[r] = mult * sum_b x_b[r] / sqrt(mean(x_b[r]^2) + eps) * w_b: several mixers' results, each normed
//                 over the row with a weight of its own, averaged
//   scale_rows    x *= c
//
// One block per row; a row is read once (it is kept in shared memory between the sum of squares and the output).
#include "common.cuh"

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w];
    return s;
}

struct StreamJoinParams {
    float* x;                 // [T, H]
    const void* delta;        // [T, H] or null
    const float* gate;        // [T, ld_gate] logits or null (delta joins ungated)
    int ld_gate;
    const float* rows_add;    // [T, H] or null
    const float* vec_add;     // [H] or null
    const float* weight;      // [H] or null: no output
    void* out;                // [T, H]
    int H;
    float eps;
};

template <typename TD, typename TO>
__global__ void __launch_bounds__(256) stream_join_kernel(StreamJoinParams p) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[8];
    const int r = blockIdx.x, H = p.H;
    llb_grid_dependency_sync();
    float* x = p.x + (size_t)r * H;
    const TD* delta = p.delta ? (const TD*)p.delta + (size_t)r * H : nullptr;
    const float* gate = p.gate ? p.gate + (size_t)r * p.ld_gate : nullptr;
    const float* ra = p.rows_add ? p.rows_add + (size_t)r * H : nullptr;
    const float* va = p.vec_add;
    const bool write = delta || ra || va;
    float ss = 0.f;
    // four elements a thread and round where the row allows it (16-byte pieces of the float32 operands)
    const bool vec = H % 4 == 0 && p.ld_gate % 4 == 0 &&
                     !(((uintptr_t)p.x | (uintptr_t)p.delta | (uintptr_t)p.gate | (uintptr_t)p.rows_add | (uintptr_t)p.vec_add) & 15);
    if (vec) {
        for (int i = threadIdx.x * 4; i < H; i += 1024) {
            float4 v = *reinterpret_cast<const float4*>(x + i);
            float* e = reinterpret_cast<float*>(&v);
            if (ra) {
                const float4 a = *reinterpret_cast<const float4*>(ra + i);
                e[0] += a.x; e[1] += a.y; e[2] += a.z; e[3] += a.w;
            }
            if (va) {
                const float4 a = *reinterpret_cast<const float4*>(va + i);
                e[0] += a.x; e[1] += a.y; e[2] += a.z; e[3] += a.w;
            }
            if (delta) {
                float d[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) d[u] = to_f32(delta[i + u]);
                if (gate) {
                    const float4 g = *reinterpret_cast<const float4*>(gate + i);
                    const float gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) d[u] = d[u] / (1.0f + expf(-gg[u]));
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) e[u] += d[u];
            }
            if (write) *reinterpret_cast<float4*>(x + i) = v;
            *reinterpret_cast<float4*>(row + i) = v;
            ss += (e[0] * e[0] + e[1] * e[1]) + (e[2] * e[2] + e[3] * e[3]);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += 256) {
            float v = x[i];
            if (ra) v += ra[i];
            if (va) v += va[i];
            if (delta) {
                const float dl = to_f32(delta[i]);
                v += gate ? dl / (1.0f + expf(-gate[i])) : dl;
            }
            if (write) x[i] = v;
            row[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    if (!p.weight) return;
    ss = block_sum_256(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + p.eps);
    const float* w = p.weight;
    TO* out = (TO*)p.out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += 256) out[i] = from_f32<TO>(row[i] * inv * w[i]);
}

LLB_API int llb_stream_join(StreamJoinParams p, int delta_dtype, int out_dtype, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    const size_t smem = (size_t)p.H * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(delta_dtype, TD, {
        LLB_DISPATCH_DTYPE(out_dtype, TO, {
            auto k = stream_join_kernel<TD, TO>;
            static bool configured = false;
            if (!configured && smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
                if (e != cudaSuccess) return (int)e;
                configured = true;
            }
            llb_launch(k, dim3(T), dim3(256), smem, stream, p);
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ mean of normed branches
struct BranchMeanParams {
    const float* x[4];        // [T, H] each
    const void* w[4];         // [H] each
    int n;
    float* out;               // [T, H]
    int H;
    float eps, mult;
};

template <typename TW>
__global__ void __launch_bounds__(256) branch_mean_kernel(BranchMeanParams p) {
    __shared__ float red[8];
    const int r = blockIdx.x, H = p.H;
    llb_grid_dependency_sync();
    float inv[4];
    for (int b = 0; b < p.n; ++b) {
        const float* x = p.x[b] + (size_t)r * H;
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += 256) ss = fmaf(x[i], x[i], ss);
        ss = block_sum_256(ss, red);
        inv[b] = 1.0f / sqrtf(ss / (float)H + p.eps);
    }
    for (int i = threadIdx.x; i < H; i += 256) {
        float acc = 0.f;
        for (int b = 0; b < p.n; ++b) acc += p.x[b][(size_t)r * H + i] * inv[b] * to_f32(((const TW*)p.w[b])[i]);
        p.out[(size_t)r * H + i] = acc * p.mult;
    }
}

LLB_API int llb_branch_mean(BranchMeanParams p, int w_dtype, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    if (p.n < 1 || p.n > 4) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(w_dtype, TW, llb_launch(branch_mean_kernel<TW>, dim3(T), dim3(256), 0, stream, p));
    return llb_status();
}

// ------------------------------------------------------------------ x *= c
__global__ void scale_rows_kernel(float* __restrict__ x, size_t n, float c) {
    llb_grid_dependency_sync();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= c;
}

LLB_API int llb_scale_rows(float* x, long long n, float c, cudaStream_t stream) {
    if (n == 0) return 0;
    llb_launch(scale_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, (size_t)n, c);
    return llb_status();
}
