// Routed experts: the router, the plan that sorts (token, choice) pairs by expert, the matrix products of the
// experts over their own tokens, and the weighted sum back into the residual stream.
//
//   select   from the router's logits z = Wr h (float32): g = 1 / (1 + e^-z); the `top` experts with the largest
//            g + bias are chosen (ties go to the lower index); a chosen expert's weight is g * route_scale, not
//            renormalised.  Mode 1: the largest logits z + bias are chosen and the weights are the softmax over the
//            chosen logits only, times route_scale.
//   plan     pair i = (token i / top, choice i % top).  Pairs are grouped by expert: slot_of[pair] is a pair's place
//            in that order, pair_of[slot] its inverse, and every expert's run of slots is cut into tiles of
//            `tile_rows` rows (tile -> expert, first slot, rows), so that the products run over a grid whose size
//            depends on the step's shape alone and never on the routing (a captured step stays valid).
//   product  out[slot, :] = act(A[row(slot), :] W[expert(slot)]^T) on the CUDA cores, float32 accumulation (the true
//            32-bit path, and the bfloat16 path wherever the tensor-core kernel below does not apply).
//   combine  stream[t, :] += sum_k weight[t, k] * y[slot_of[t top + k], :], k in order: deterministic.
#include "common.cuh"

constexpr int MOE_TILE = 64;

// ------------------------------------------------------------------ router: gates and choice from the logits
// z [T, E] are the router's logits in float32 (a matrix product of the activations with the router's matrix, float32
// accumulation).  A warp per token: gates g = 1 / (1 + e^-z), choice scores g + bias, the `top` largest by repeated
// arg-max (ties to the lower index), weights g * route_scale.
__global__ void __launch_bounds__(128)
moe_select_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, int T, int E, int top, float route_scale,
                  int* __restrict__ idx, float* __restrict__ wgt, int mode, int n_groups, int keep_groups, int renorm) {
    extern __shared__ float sm[];                 // per warp: gate[E], choice[E]
    __shared__ float group_score[4][64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    float* gate = sm + (size_t)warp * 2 * E;
    float* choice = gate + E;
    llb_grid_dependency_sync();
    if (t >= T) return;
    for (int e = lane; e < E; e += 32) {
        const float zl = z[(size_t)t * ldz + e];
        const float g = mode == 1 ? zl : 1.0f / (1.0f + expf(-zl));
        gate[e] = g;
        choice[e] = g + (bias ? bias[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 1) {
        // the experts form n_groups equal groups of neighbours; a group's score is the sum of its two largest choice
        // scores; only experts of the keep_groups best groups (first maximum first) stay in the choice
        const int per = E / n_groups;
        float* gs = group_score[warp];
        for (int g = lane; g < n_groups; g += 32) {
            float b0 = -INFINITY, b1 = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float c = choice[e];
                if (c > b0) { b1 = b0; b0 = c; }
                else if (c > b1) b1 = c;
            }
            gs[g] = per > 1 ? b0 + b1 : b0;
        }
        __syncwarp();
        if (lane == 0) {
            for (int k = 0; k < keep_groups; ++k) {
                int arg = -1;
                float best = -INFINITY;
                for (int g = 0; g < n_groups; ++g)
                    if (gs[g] != INFINITY && (arg < 0 || gs[g] > best)) { best = gs[g]; arg = g; }
                if (arg >= 0) gs[arg] = INFINITY;          // kept
            }
        }
        __syncwarp();
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; arg = e; }          // ascending e: the first maximum of this lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) {                           // every score left is NaN or -inf: the lowest index not taken yet
            arg = 0;
            while (arg < E - 1 && choice[arg] == -INFINITY) ++arg;
        }
        if (lane == 0) {
            idx[(size_t)t * top + k] = arg;
            wgt[(size_t)t * top + k] = mode == 1 ? gate[arg] : gate[arg] * route_scale;
            choice[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (mode == 1 && lane == 0) {
        // softmax over the chosen logits only, in the order they were chosen
        float* w = wgt + (size_t)t * top;
        float mx = -INFINITY;
        for (int k = 0; k < top; ++k) mx = fmaxf(mx, w[k]);
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const float ex = expf(w[k] - mx);
            w[k] = ex;
            sum += ex;
        }
        const float inv = route_scale / sum;
        for (int k = 0; k < top; ++k) w[k] *= inv;
    }
    if (mode != 1 && renorm && lane == 0) {
        // the chosen gates divided by their sum (the factor route_scale is in them already)
        float* w = wgt + (size_t)t * top;
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += w[k];
        const float inv = route_scale / (sum + 1e-20f * route_scale);
        for (int k = 0; k < top; ++k) w[k] *= inv;
    }
}

LLB_API int llb_moe_select(const float* z, int ldz, const float* bias, int T, int E, int top, float route_scale, int* idx,
                           float* wgt, int mode, int n_groups, int keep_groups, int renorm, cudaStream_t stream) {
    if (T == 0) return 0;
    if (top < 1 || top > E) return (int)cudaErrorInvalidValue;
    if (n_groups > 1 && (n_groups > 64 || E % n_groups || keep_groups < 1 || keep_groups > n_groups)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    llb_launch(moe_select_kernel, dim3((T + 3) / 4), dim3(128), smem, stream, z, ldz, bias, T, E, top, route_scale, idx, wgt, mode,
               n_groups, keep_groups, renorm);
    return llb_status();
}

// ------------------------------------------------------------------ plan
// One block.  tiles: int32 [3, max_tiles] (expert, first slot, rows) and n_tiles [1]; max_tiles >= N / tile_rows + min(E, N).
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ idx, int N, int E, int tile_rows, int* __restrict__ slot_of, int* __restrict__ pair_of,
                int* __restrict__ tiles, int max_tiles, int* __restrict__ n_tiles) {
    extern __shared__ int si[];                   // count[E], first[E], cursor[E], tile0[E + 1]
    int* count = si;
    int* first = count + E;
    int* cursor = first + E;
    int* tile0 = cursor + E;
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
    llb_grid_dependency_sync();
    __syncthreads();
    // (four pairs per thread and round: the block is alone on the device, so its loads have to be in flight together)
    for (int i0 = tid; i0 < N; i0 += 4 * blockDim.x) {
        int e4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) e4[u] = i0 + u * blockDim.x < N ? idx[i0 + u * blockDim.x] : -1;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (e4[u] >= 0 && e4[u] < E) atomicAdd(&count[e4[u]], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int f = 0, tl = 0;
        for (int e = 0; e < E; ++e) {
            first[e] = f;
            tile0[e] = tl;
            f += count[e];
            tl += (count[e] + tile_rows - 1) / tile_rows;
        }
        tile0[E] = tl;
        *n_tiles = min(tl, max_tiles);
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
        for (int i = tile0[e], r = 0; i < tile0[e + 1] && i < max_tiles; ++i, r += tile_rows) {
            tiles[i] = e;
            tiles[max_tiles + i] = first[e] + r;
            tiles[2 * max_tiles + i] = min(tile_rows, count[e] - r);
        }
    }
    for (int i0 = tid; i0 < N; i0 += 4 * blockDim.x) {
        int e4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) e4[u] = i0 + u * blockDim.x < N ? idx[i0 + u * blockDim.x] : -1;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e4[u], i = i0 + u * blockDim.x;
            if (e < 0 || e >= E) continue;
            const int s = first[e] + atomicAdd(&cursor[e], 1);
            slot_of[i] = s;
            pair_of[s] = i;
        }
    }
}

LLB_API int llb_moe_plan(const int* idx, int N, int E, int tile_rows, int* slot_of, int* pair_of, int* tiles, int max_tiles,
                         int* n_tiles, cudaStream_t stream) {
    if (N == 0) return 0;
    const size_t smem = (size_t)(4 * E + 1) * sizeof(int);
    if (tile_rows < 1 || smem > 48 * 1024 || max_tiles < N / tile_rows + (E < N ? E : N)) return (int)cudaErrorInvalidValue;
    llb_launch(moe_plan_kernel, dim3(1), dim3(1024), smem, stream, idx, N, E, tile_rows, slot_of, pair_of, tiles, max_tiles, n_tiles);
    return llb_status();
}

// the most rows of a tile that the CUDA-core product below takes
LLB_API int llb_moe_tile_rows() { return MOE_TILE; }

// ------------------------------------------------------------------ the experts' products on the CUDA cores
// out[slot, n] = act(sum_k A[row(slot), k] W[expert][n, k]) for the slots of one tile; row(slot) = pair_of[slot] / top
// when the rows are gathered from the tokens (GATHER), else slot itself.  ACT 1: max(., 0)^2; 2: gelu (erf form).
template <typename TA, typename TW, typename TO, bool GATHER, int ACT>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ pair_of, int top, const TW* __restrict__ W,
                TO* __restrict__ out, int ldo, const int* __restrict__ tiles, int max_tiles, const int* __restrict__ n_tiles,
                int N, int K) {
    constexpr int BM = MOE_TILE, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int rows_s[BM];
    llb_grid_dependency_sync();
    const int tile = blockIdx.y;
    if (tile >= *n_tiles) return;
    const int e = tiles[tile], slot0 = tiles[max_tiles + tile], rows = tiles[2 * max_tiles + tile];
    const int tid = threadIdx.x, n0 = blockIdx.x * BN;
    if (tid < BM) rows_s[tid] = tid < rows ? (GATHER ? pair_of[slot0 + tid] / top : slot0 + tid) : -1;
    __syncthreads();
    const TW* We = W + (size_t)e * N * K;
    const int ty = tid / 16, tx = tid % 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int lr = tid / 4, lk = (tid % 4) * 4;
    const int arow = rows_s[lr];
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q, n = n0 + lr;
            As[lk + q][lr] = (arow >= 0 && k < K) ? to_f32(A[(size_t)arow * lda + k]) : 0.f;
            Ws[lk + q][lr] = (n < N && k < K) ? to_f32(We[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (ACT == 1) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            if (ACT == 2) v = 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
            out[(size_t)(slot0 + r) * ldo + n] = from_f32<TO>(v);
        }
    }
}

// gather != 0: A is the tokens' activations [T, lda] and a slot's row is its pair's token; else A is [slots, lda].
// act 1: squared ReLU, 2: gelu (erf form).  W is the experts' matrices stacked, [E, N, K].
LLB_API int llb_moe_gemm(const void* A, int a_dtype, int lda, const int* pair_of, int top, int gather, const void* W,
                         int w_dtype, void* out, int o_dtype, int ldo, const int* tiles, int max_tiles, const int* n_tiles,
                         int N, int K, int act, cudaStream_t stream) {
    if (max_tiles == 0 || N == 0) return 0;
    if (max_tiles > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((N + 63) / 64, max_tiles);
#define LLB_MG(G, ACT)                                                                                                  \
    llb_launch(moe_gemm_kernel<TA, TW, TO, G, ACT>, grid, dim3(256), 0, stream, (const TA*)A, lda, pair_of, top,        \
               (const TW*)W, (TO*)out, ldo, tiles, max_tiles, n_tiles, N, K)
    LLB_DISPATCH_DTYPE(a_dtype, TA, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            LLB_DISPATCH_DTYPE(o_dtype, TO, {
                if (gather && act == 1) LLB_MG(true, 1);
                else if (gather && act == 2) LLB_MG(true, 2);
                else if (gather) LLB_MG(true, 0);
                else if (act == 1) LLB_MG(false, 1);
                else if (act == 2) LLB_MG(false, 2);
                else LLB_MG(false, 0);
            });
        });
    });
#undef LLB_MG
    return llb_status();
}

// ------------------------------------------------------------------ the tokens' rows in slot order
// out[slot, :] = x[pair_of[slot] / top, :]: the activations as the tensor-core product wants them (a tile's rows in one
// box).  16-byte pieces where the rows allow it.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ pair_of, int top, T* __restrict__ out, int H) {
    llb_grid_dependency_sync();
    const int slot = blockIdx.x;
    const T* src = x + (size_t)(pair_of[slot] / top) * ldx;
    T* dst = out + (size_t)slot * H;
    constexpr int V = 16 / sizeof(T);
    if (H % V == 0 && ldx % V == 0 && !(((uintptr_t)x | (uintptr_t)out) & 15)) {
        for (int j = threadIdx.x; j < H / V; j += blockDim.x)
            reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(src)[j];
    } else {
        for (int j = threadIdx.x; j < H; j += blockDim.x) dst[j] = src[j];
    }
}

LLB_API int llb_moe_gather_rows(const void* x, int dtype, int ldx, const int* pair_of, int top, void* out, int n_slots, int H,
                                cudaStream_t stream) {
    if (n_slots == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, T,
        llb_launch(moe_gather_rows_kernel<T>, dim3(n_slots), dim3(256), 0, stream, (const T*)x, ldx, pair_of, top, (T*)out, H));
    return llb_status();
}

// ------------------------------------------------------------------ weighted sum into the stream
template <typename TY>
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ stream, const TY* __restrict__ y, int ldy, const int* __restrict__ slot_of,
                   const float* __restrict__ wgt, int top, int H) {
    llb_grid_dependency_sync();
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k)
            acc = fmaf(wgt[(size_t)t * top + k], to_f32(y[(size_t)slot_of[(size_t)t * top + k] * ldy + j]), acc);
        stream[(size_t)t * H + j] += acc;
    }
}

LLB_API int llb_moe_combine(float* stream, const void* y, int y_dtype, int ldy, const int* slot_of, const float* wgt, int T,
                            int top, int H, cudaStream_t stream_) {
    if (T == 0) return 0;
    LLB_DISPATCH_DTYPE(y_dtype, TY,
        llb_launch(moe_combine_kernel<TY>, dim3(T), dim3(256), 0, stream_, stream, (const TY*)y, ldy, slot_of, wgt, top, H));
    return llb_status();
}
