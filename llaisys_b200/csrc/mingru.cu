// The minGRU recurrence: a gated recurrence per channel whose gates read the current token only,
//
//     z_t = sigmoid(a_t)            c_t = u_t + 1/2 (u_t >= 0),  sigmoid(u_t) (u_t < 0)
//     S_t = (1 - z_t) S_{t-1} + z_t c_t            y_t = S_t * silu(g_t)
//
// over the new tokens of every sequence of a step.  proj [T, ld] holds the step's projections (biases included): the
// gate logits a at column a_off, the candidate inputs u at u_off, the output gate g at g_off, `width` columns each.
// state [slots, width] (float32) is read at row seq_slot[b] and left holding S after the sequence's last token.
// Gates, candidates, the state and its sums are float32 whatever the projections' type.
//
// Since S_t is an affine function of S_{t-1}, a stretch of tokens composes into one pair (A, B) with
// S_end = A S_start + B.  Short steps (up to `chunk` tokens a sequence) run one thread per (sequence, channel) over
// the tokens in order.  Longer ones are cut into chunks of `chunk` tokens: mingru_reduce forms (A, B) of every chunk,
// mingru_prefix walks a sequence's chunks in order (the state each chunk starts from; the sequence's last state), and
// mingru_apply runs every chunk from its start state and writes y: the tokens of a long prompt are worked on by
// T / chunk threads a channel instead of one.  The walk over the chunks and the order inside a chunk are fixed, so a
// token's result does not depend on what else the step holds.
#include "common.cuh"

struct MinGruParams {
    const void* proj;         // [T, ld]
    int ld, a_off, u_off, g_off, width;
    float* state;             // [slots, width]
    const int* seq_start;     // [B + 1]
    const int* seq_slot;      // [B]
    void* out;                // [T, width]
    float* chunk_a;           // [B, n_chunks, width]: A of a chunk, then (after the prefix pass) the state it starts from
    float* chunk_b;           // [B, n_chunks, width]
    int chunk, n_chunks;
};

#define MG_AHEAD 8            // tokens whose loads a thread has in flight

__device__ __forceinline__ float mg_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float mg_candidate(float u) { return u >= 0.f ? u + 0.5f : mg_sigmoid(u); }

// One thread per (sequence, channel): tokens t0 .. t1 of the sequence in order from state S; returns the last state.
template <typename TI, typename TO, bool WRITE>
__device__ __forceinline__ float mg_run(const MinGruParams& p, int ch, int t0, int t1, float S) {
    const TI* proj = (const TI*)p.proj;
    TO* out = (TO*)p.out;
    int t = t0;
    // eight tokens' loads are requested before the first is used: the recurrence itself is a few dependent operations,
    // and a long prompt's chunks fill only part of the SMs' warps
    for (; t + MG_AHEAD <= t1; t += MG_AHEAD) {
        float a[MG_AHEAD], u[MG_AHEAD], g[MG_AHEAD];
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) {
            const TI* row = proj + (size_t)(t + i) * p.ld;
            a[i] = to_f32(row[p.a_off + ch]);
            u[i] = to_f32(row[p.u_off + ch]);
            if (WRITE) g[i] = to_f32(row[p.g_off + ch]);
        }
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) {
            const float z = mg_sigmoid(a[i]);
            S = fmaf(z, mg_candidate(u[i]) - S, S);            // (1 - z) S + z c
            if (WRITE) out[(size_t)(t + i) * p.width + ch] = from_f32<TO>(S * g[i] * mg_sigmoid(g[i]));
        }
    }
    for (; t < t1; ++t) {
        const TI* row = proj + (size_t)t * p.ld;
        const float z = mg_sigmoid(to_f32(row[p.a_off + ch]));
        S = fmaf(z, mg_candidate(to_f32(row[p.u_off + ch])) - S, S);
        if (WRITE) {
            const float g = to_f32(row[p.g_off + ch]);
            out[(size_t)t * p.width + ch] = from_f32<TO>(S * g * mg_sigmoid(g));
        }
    }
    return S;
}

// short steps: grid (channel blocks, B)
template <typename TI, typename TO>
__global__ void __launch_bounds__(128) mingru_scan_kernel(MinGruParams p) {
    const int ch = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
    llb_grid_dependency_sync();
    if (ch >= p.width) return;
    const int t0 = p.seq_start[b], t1 = p.seq_start[b + 1];
    if (t1 <= t0) return;
    float* st = p.state + (size_t)p.seq_slot[b] * p.width + ch;
    *st = mg_run<TI, TO, true>(p, ch, t0, t1, *st);
}

// (A, B) of every chunk: grid (channel blocks, n_chunks, B)
template <typename TI>
__global__ void __launch_bounds__(128) mingru_reduce_kernel(MinGruParams p) {
    const int ch = blockIdx.x * 128 + threadIdx.x, k = blockIdx.y, b = blockIdx.z;
    llb_grid_dependency_sync();
    if (ch >= p.width) return;
    const int s0 = p.seq_start[b], s1 = p.seq_start[b + 1];
    const int t0 = s0 + k * p.chunk, t1 = min(s1, t0 + p.chunk);
    if (t0 >= s1) return;
    const TI* proj = (const TI*)p.proj;
    float A = 1.f, B = 0.f;
    int t = t0;
    for (; t + MG_AHEAD <= t1; t += MG_AHEAD) {
        float a[MG_AHEAD], u[MG_AHEAD];
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) {
            const TI* row = proj + (size_t)(t + i) * p.ld;
            a[i] = to_f32(row[p.a_off + ch]);
            u[i] = to_f32(row[p.u_off + ch]);
        }
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) {
            const float z = mg_sigmoid(a[i]);
            A *= 1.f - z;
            B = fmaf(z, mg_candidate(u[i]) - B, B);
        }
    }
    for (; t < t1; ++t) {
        const TI* row = proj + (size_t)t * p.ld;
        const float z = mg_sigmoid(to_f32(row[p.a_off + ch]));
        A *= 1.f - z;
        B = fmaf(z, mg_candidate(to_f32(row[p.u_off + ch])) - B, B);
    }
    const size_t i = ((size_t)b * p.n_chunks + k) * p.width + ch;
    p.chunk_a[i] = A;
    p.chunk_b[i] = B;
}

// the state every chunk starts from (into chunk_a), and the sequence's last state: grid (channel blocks, B)
__global__ void __launch_bounds__(128) mingru_prefix_kernel(MinGruParams p) {
    const int ch = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
    llb_grid_dependency_sync();
    if (ch >= p.width) return;
    const int n_new = p.seq_start[b + 1] - p.seq_start[b];
    if (n_new <= 0) return;
    const int chunks = (n_new + p.chunk - 1) / p.chunk;
    float* st = p.state + (size_t)p.seq_slot[b] * p.width + ch;
    float S = *st;
    const size_t base = (size_t)b * p.n_chunks * p.width + ch;
    int k = 0;
    // eight chunks' pairs are fetched together (the walk itself is one multiply-add a chunk, a load's latency each otherwise)
    for (; k + 8 <= chunks; k += 8) {
        float A[8], B[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            A[j] = p.chunk_a[base + (size_t)(k + j) * p.width];
            B[j] = p.chunk_b[base + (size_t)(k + j) * p.width];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            p.chunk_a[base + (size_t)(k + j) * p.width] = S;
            S = fmaf(A[j], S, B[j]);
        }
    }
    for (; k < chunks; ++k) {
        const size_t i = base + (size_t)k * p.width;
        const float A = p.chunk_a[i], B = p.chunk_b[i];
        p.chunk_a[i] = S;
        S = fmaf(A, S, B);
    }
    *st = S;
}

// every chunk from its start state: grid (channel blocks, n_chunks, B)
template <typename TI, typename TO>
__global__ void __launch_bounds__(128) mingru_apply_kernel(MinGruParams p) {
    const int ch = blockIdx.x * 128 + threadIdx.x, k = blockIdx.y, b = blockIdx.z;
    llb_grid_dependency_sync();
    if (ch >= p.width) return;
    const int s0 = p.seq_start[b], s1 = p.seq_start[b + 1];
    const int t0 = s0 + k * p.chunk, t1 = min(s1, t0 + p.chunk);
    if (t0 >= s1) return;
    mg_run<TI, TO, true>(p, ch, t0, t1, p.chunk_a[((size_t)b * p.n_chunks + k) * p.width + ch]);
}

// n_chunks = ceil(max_new / chunk); 1 (or no scratch): every sequence runs in one go
LLB_API int llb_mingru(MinGruParams p, int in_dtype, int out_dtype, int B, cudaStream_t stream) {
    if (B == 0 || p.width == 0) return 0;
    const unsigned cb = (unsigned)((p.width + 127) / 128);
    if (B > 65535 || p.n_chunks > 65535) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(in_dtype, TI, {
        LLB_DISPATCH_DTYPE(out_dtype, TO, {
            if (p.n_chunks <= 1 || !p.chunk_a || !p.chunk_b) {
                llb_launch(mingru_scan_kernel<TI, TO>, dim3(cb, B), dim3(128), 0, stream, p);
                return llb_status();
            }
            llb_launch(mingru_reduce_kernel<TI>, dim3(cb, p.n_chunks, B), dim3(128), 0, stream, p);
            llb_launch(mingru_prefix_kernel, dim3(cb, B), dim3(128), 0, stream, p);
            llb_launch(mingru_apply_kernel<TI, TO>, dim3(cb, p.n_chunks, B), dim3(128), 0, stream, p);
        });
    });
    return llb_status();
}
