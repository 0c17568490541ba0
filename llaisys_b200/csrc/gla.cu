// Gated linear attention: a recurrent mixer whose memory per head is a matrix S [key channels, value channels] in
// float32, decayed per key channel and updated by an outer product at every token:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,      a_t = sigmoid(z_t)^(1/tau)
//
// The state row of a sequence lives in the cache's fixed-size state table ([slots, heads * dk * dv]) and is carried
// from step to step; one kernel serves a whole prompt, a portion of one and a single token (it walks the new tokens of
// its sequence in order).  Everything that enters the recurrence besides the projections q, k, v is float32: the decay
// logits z arrive in float32, a = exp(-softplus(-z) / tau) is formed here, the state and the sums stay float32.
//
//  * gla_scan: a block owns a group of value columns of one head of one sequence; 4, 8 or 16 lanes share a column, each
//    with a run of its key channels (KPT state values in registers); q, k, a and v of sixteen tokens at a time are
//    staged in shared memory, the next sixteen being fetched into registers meanwhile; the chunk runs without a branch
//    and every o_t is completed by shuffles among the lanes of its column, those of a chunk together.
//  * gla_out: per (token, head) one warp: RMS norm of o over the value channels with a weight shared by the heads,
//    times silu of the output gate.
#include "common.cuh"

constexpr int GLA_THREADS = 128;
constexpr int GLA_CHUNK = 16;     // tokens staged at a time

struct GlaParams {
    const void* q;            // packed projections [T, row_stride]: head h's queries at q + h * dk
    const void* k;            // the same buffer at its first key column
    const void* v;            // the same buffer at its first value column
    int row_stride;
    const float* z;           // decay logits [T, z_stride], head h at h * dk (z_is_decay: the decays themselves)
    int z_stride;
    float* state;             // [slots, H * dk * dv]
    const int* seq_start;     // [B + 1]
    const int* seq_slot;      // [B]
    float* out;               // [T, H * dv]
    int H, dk, dv;
    float q_scale, inv_tau;
    int z_is_decay;           // z already holds a = sigmoid(z)^(1/tau) (llb_gla_decay ran over it)
    const float* head_decay;  // [H] or null: one constant decay a head, the same for every token and key channel (z is not read)
    int act;                  // 1: q, k and v pass through silu on their way in
};

// log sigmoid(z) = -softplus(-z) = -(max(-z, 0) + log(1 + e^-|z|));  a = sigmoid(z)^(1/tau) = exp(log sigmoid(z) / tau)
__device__ __forceinline__ float gla_decay(float z, float inv_tau) {
    return expf(-(fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)))) * inv_tau);
}

// z <- a in place, once per (token, channel): for many tokens, so that the blocks that share a head do not each repeat it.
__global__ void gla_decay_kernel(float* __restrict__ z, size_t n, float inv_tau) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z[i] = gla_decay(z[i], inv_tau);
}

LLB_API int llb_gla_decay(float* z, long long n, float inv_tau, cudaStream_t stream) {
    if (n == 0) return 0;
    llb_launch(gla_decay_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, (size_t)n, inv_tau);
    return llb_status();
}

// KS lanes share a value column, each with KPT consecutive key channels of it (KPT a multiple of 4); a block of 128
// threads owns 128 / KS columns.  In shared memory a lane's channels of a token are KPT consecutive floats, the lanes'
// groups an odd number of 16-byte pieces apart, so that the 16-byte reads of the lanes of a quarter-warp fall on
// different banks (measured with groups 32 bytes apart: two-way conflicts on every read of q, k and a).
constexpr int gla_pad(int kpt) { return (kpt / 4) % 2 == 1 ? 0 : 4; }
template <typename T, int KS, int KPT>
__global__ void __launch_bounds__(GLA_THREADS) gla_scan_kernel(GlaParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int COLS = GLA_THREADS / KS;
    constexpr int DKP = KS * KPT;                     // key channels, padded
    constexpr int PAD = gla_pad(KPT);
    constexpr int ROW = KS * (KPT + PAD);               // floats of one token's q (or k, or a) in shared memory
    float* sq = sm;                                   // [CHUNK][ROW]
    float* sk = sq + GLA_CHUNK * ROW;
    float* sa = sk + GLA_CHUNK * ROW;
    float* sv = sa + GLA_CHUNK * ROW;                 // [CHUNK][COLS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = lane & (KS - 1), jl = lane / KS;
    const int cloc = warp * (32 / KS) + jl;           // column within the block
    const int col = blockIdx.x * COLS + cloc;
    const int h = blockIdx.y, b = blockIdx.z;
    const int dk = p.dk, dv = p.dv;
    llb_grid_dependency_sync();
    const int tok0 = p.seq_start[b], n = p.seq_start[b + 1] - tok0;
    float* st = p.state + ((size_t)p.seq_slot[b] * p.H + h) * dk * dv;
    float S[KPT];
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
        int i = part * KPT + m;
        S[m] = (i < dk && col < dv) ? st[(size_t)i * dv + col] : 0.f;
    }
    const T* qb = (const T*)p.q;
    const T* kb = (const T*)p.k;
    const T* vb = (const T*)p.v;
    // A chunk's q, k, z and v are fetched into registers while the chunk before it is computed, and pass through the
    // decay's arithmetic into shared memory when their turn comes: the walk never waits for a load it has just issued.
    constexpr int NQ = (GLA_CHUNK * DKP + GLA_THREADS - 1) / GLA_THREADS;
    constexpr int NV = (GLA_CHUNK * COLS + GLA_THREADS - 1) / GLA_THREADS;
    float rq[NQ], rk[NQ], rz[NQ], rv[NV];
    const bool is_decay = p.z_is_decay || p.head_decay;
    const float head_a = p.head_decay ? p.head_decay[h] : 0.f;
    auto act = [&](float x) { return p.act == 1 ? x / (1.0f + expf(-x)) : x; };
    auto fetch = [&](int c0) {
        const int nc = min(GLA_CHUNK, n - c0);
#pragma unroll
        for (int e = 0; e < NQ; ++e) {
            const int idx = tid + e * GLA_THREADS, t = idx / DKP, i = idx - t * DKP;
            rq[e] = rk[e] = 0.f;
            rz[e] = is_decay ? 1.f : INFINITY;             // a decay of exactly one
            if (idx < GLA_CHUNK * DKP && i < dk && t < nc) {
                const size_t row = (size_t)(tok0 + c0 + t);
                rq[e] = act(to_f32(qb[row * p.row_stride + h * dk + i]));
                rk[e] = act(to_f32(kb[row * p.row_stride + h * dk + i]));
                rz[e] = p.head_decay ? head_a : p.z[row * p.z_stride + h * dk + i];
            }
        }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = tid + e * GLA_THREADS, t = idx / COLS, c = idx - t * COLS;
            const int cc = blockIdx.x * COLS + c;
            rv[e] = (idx < GLA_CHUNK * COLS && cc < dv && t < nc) ? act(to_f32(vb[(size_t)(tok0 + c0 + t) * p.row_stride + h * dv + cc])) : 0.f;
        }
    };
    fetch(0);
    for (int c0 = 0; c0 < n; c0 += GLA_CHUNK) {
        const int nc = min(GLA_CHUNK, n - c0);
        __syncthreads();
        // (token slots past the step's end hold a = 1, k = 0, q = 0: they leave the state as it is, so the tokens of a
        // chunk run without a branch and their reductions overlap)
#pragma unroll
        for (int e = 0; e < NQ; ++e) {
            const int idx = tid + e * GLA_THREADS;
            if (idx < GLA_CHUNK * DKP) {
                const int t = idx / DKP, i = idx - t * DKP;
                const int at = t * ROW + (i / KPT) * (KPT + PAD) + (i % KPT);
                sq[at] = rq[e] * p.q_scale;
                sk[at] = rk[e];
                sa[at] = is_decay ? rz[e] : gla_decay(rz[e], p.inv_tau);
            }
        }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = tid + e * GLA_THREADS;
            if (idx < GLA_CHUNK * COLS) sv[idx] = rv[e];
        }
        __syncthreads();
        if (c0 + GLA_CHUNK < n) fetch(c0 + GLA_CHUNK);
        float acc[GLA_CHUNK];
#pragma unroll
        for (int t = 0; t < GLA_CHUNK; ++t) {
            const float vv = sv[t * COLS + cloc];
            const float4* a4 = reinterpret_cast<const float4*>(sa + t * ROW + part * (KPT + PAD));
            const float4* k4 = reinterpret_cast<const float4*>(sk + t * ROW + part * (KPT + PAD));
            const float4* q4 = reinterpret_cast<const float4*>(sq + t * ROW + part * (KPT + PAD));
            float a0 = 0.f, a1 = 0.f;                 // two chains, so that the sum does not wait on one
#pragma unroll
            for (int m = 0; m < KPT; m += 4) {
                const float4 a = a4[m / 4], k = k4[m / 4], q = q4[m / 4];
                S[m] = fmaf(a.x, S[m], k.x * vv);
                a0 = fmaf(S[m], q.x, a0);
                S[m + 1] = fmaf(a.y, S[m + 1], k.y * vv);
                a1 = fmaf(S[m + 1], q.y, a1);
                S[m + 2] = fmaf(a.z, S[m + 2], k.z * vv);
                a0 = fmaf(S[m + 2], q.z, a0);
                S[m + 3] = fmaf(a.w, S[m + 3], k.w * vv);
                a1 = fmaf(S[m + 3], q.w, a1);
            }
            acc[t] = a0 + a1;
        }
#pragma unroll
        for (int o = 1; o < KS; o <<= 1) {
#pragma unroll
            for (int t = 0; t < GLA_CHUNK; ++t) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
        }
        if (part == 0 && col < dv) {
#pragma unroll
            for (int t = 0; t < GLA_CHUNK; ++t)
                if (t < nc) p.out[(size_t)(tok0 + c0 + t) * p.H * dv + h * dv + col] = acc[t];
        }
    }
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
        int i = part * KPT + m;
        if (i < dk && col < dv) st[(size_t)i * dv + col] = S[m];
    }
}

template <typename T, int KS, int KPT>
static int launch_scan(const GlaParams& p, int B, cudaStream_t stream) {
    auto k = gla_scan_kernel<T, KS, KPT>;
    constexpr int COLS = GLA_THREADS / KS;
    constexpr int PAD = gla_pad(KPT);
    size_t smem = (size_t)(3 * GLA_CHUNK * KS * (KPT + PAD) + GLA_CHUNK * COLS) * sizeof(float);
    dim3 grid((p.dv + COLS - 1) / COLS, p.H, B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    static bool configured = false;          // once per instantiation: not repeated inside a graph capture
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    configured = true;
    llb_launch(k, grid, dim3(GLA_THREADS), smem, stream, p);
    return llb_status();
}

template <typename T, int KS>
static int launch_scan_ks(const GlaParams& p, int B, cudaStream_t stream) {
    const int kpt = (p.dk + KS - 1) / KS;
    if (kpt <= 4) return launch_scan<T, KS, 4>(p, B, stream);
    if (kpt <= 8) return launch_scan<T, KS, 8>(p, B, stream);
    if (kpt <= 16) return launch_scan<T, KS, 16>(p, B, stream);
    if constexpr (KS <= 8) {
        if (kpt <= 32) return launch_scan<T, KS, 32>(p, B, stream);
    }
    if constexpr (KS <= 4) {
        if (kpt <= 64) return launch_scan<T, KS, 64>(p, B, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// Runs the recurrence over the new tokens of every sequence of the step and writes o [T, H * dv] (float32).
// sms: multiprocessors of the device.  More lanes share a column (fewer columns a block, more blocks) while the blocks
// would not fill the device and a lane still keeps four channels or more.  (Measured and lost at 32 heads of 128 x 128
// over 2,048 tokens, 800 us as it is: splitting further, 16 lanes a column, 867 us; four columns a lane, so that what a
// lane reads of q, k and a serves four columns, 1,129 us with a quarter of the blocks.  The walk is bound by latency
// at one warp a scheduler, about 120 instructions a token and warp, not by shared memory or arithmetic.)
LLB_API int llb_gla_scan(GlaParams p, int dtype, int B, int sms, cudaStream_t stream) {
    if (B == 0) return 0;
    if (p.dk <= 0 || p.dv <= 0 || p.H <= 0 || p.dk > 256) return (int)cudaErrorInvalidValue;
    int ks = 4;
    while (ks < 16 && (long long)((p.dv + 128 / ks - 1) / (128 / ks)) * p.H * B < sms && p.dk >= 8 * ks) ks *= 2;
    LLB_DISPATCH_DTYPE(dtype, T, {
        if (ks == 4) return launch_scan_ks<T, 4>(p, B, stream);
        if (ks == 8) return launch_scan_ks<T, 8>(p, B, stream);
        return launch_scan_ks<T, 16>(p, B, stream);
    });
    return 0;
}

// ------------------------------------------------------------------ long steps with a constant decay per head, chunk by chunk
// With one decay a_h per head the state after a run of n tokens is a_h^n S_before + (the state the run reaches from zero), so a
// long step is cut into chunks that run side by side: the recurrence over every chunk from a zero state (its local state),
// this kernel, and the recurrence again over every chunk from the state it really starts with.  Here, per sequence and state
// element: carry = the sequence's state; for each of its chunks in order, tmp[chunk] (the local state) is replaced by carry
// (what the chunk starts with) and carry <- a_h^len carry + local; at the end the sequence's state is carry.
__global__ void __launch_bounds__(256)
gla_chunk_prefix_kernel(float* __restrict__ tmp, float* __restrict__ state, const int* __restrict__ seq_chunk0,
                        const int* __restrict__ chunk_len, const int* __restrict__ seq_slot, const float* __restrict__ head_decay,
                        int per_head, int n_state) {
    llb_grid_dependency_sync();
    const int e = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (e >= n_state) return;
    const float a = head_decay[e / per_head];
    float* st = state + (size_t)seq_slot[b] * n_state + e;
    float carry = *st;
    for (int c = seq_chunk0[b]; c < seq_chunk0[b + 1]; ++c) {
        float* t = tmp + (size_t)c * n_state + e;
        const float local = *t;
        *t = carry;
        float f = 1.f;
        for (int i = 0; i < chunk_len[c]; ++i) f *= a;
        carry = fmaf(f, carry, local);
    }
    *st = carry;
}

LLB_API int llb_gla_chunk_prefix(float* tmp, float* state, const int* seq_chunk0, const int* chunk_len, const int* seq_slot,
                                 const float* head_decay, int per_head, int n_state, int B, cudaStream_t stream) {
    if (B == 0 || n_state == 0) return 0;
    if (B > 65535) return (int)cudaErrorInvalidValue;
    llb_launch(gla_chunk_prefix_kernel, dim3((n_state + 255) / 256, B), dim3(256), 0, stream, tmp, state, seq_chunk0, chunk_len,
               seq_slot, head_decay, per_head, n_state);
    return llb_status();
}

// out[t, h * dv + d] = o[t, h, d] / sqrt(mean_d o[t, h, :]^2 + eps) * w[d] * silu(g[t, h * dv + d])      (gate_act 1: sigmoid(g))
template <typename T, typename TW>
__global__ void __launch_bounds__(128) gla_out_kernel(const float* __restrict__ o, const T* __restrict__ g, int g_stride,
                                                      const TW* __restrict__ w, T* __restrict__ out, int rows, int H, int dv,
                                                      float eps, int gate_act) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);       // (token, head)
    llb_grid_dependency_sync();
    if (r >= rows) return;
    const int t = r / H, h = r - t * H;
    const float* x = o + (size_t)r * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) ss += x[d] * x[d];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
        float gv = to_f32(g[(size_t)t * g_stride + h * dv + d]);
        const float sg = 1.0f / (1.0f + expf(-gv));
        out[(size_t)r * dv + d] = from_f32<T>(x[d] * inv * to_f32(w[d]) * (gate_act == 1 ? sg : gv * sg));
    }
}

LLB_API int llb_gla_out(const float* o, const void* g, int g_stride, const void* w, int w_dtype, void* out, int dtype,
                        int T, int H, int dv, float eps, int gate_act, cudaStream_t stream) {
    int rows = T * H;
    if (rows == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            llb_launch(gla_out_kernel<TT, TW>, dim3((rows + 3) / 4), dim3(128), 0, stream, o, (const TT*)g, g_stride,
                       (const TW*)w, (TT*)out, rows, H, dv, eps, gate_act);
        });
    });
    return llb_status();
}
