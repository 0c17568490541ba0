// Causal grouped-query attention over the paged cache on the CUDA cores, float32 arithmetic.
// It serves the true 32-bit path in both phases and is the reference the tensor-core kernels
// are checked against.  Compiled per head size: -DLLB_HEAD_DIM=<at most 256> (and -DLLB_VALUE_DIM for values of another width).
//
// Formula (src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112 of xsmccc/llaisys): for a
// query at absolute position p of head h, scores s_t = (q . k_t) * scale over the keys t of kv
// head h / (nh / nkvh) with t <= p; softmax with the maximum subtracted; out = sum_t p_t v_t.
// A window W > 0 (not in that project) further restricts the keys to p - W < t <= p; with keep_first F > 0
// the keys t < F stay visible behind the window (at their true positions).  With `sink` the softmax has one
// more term of score 0 that carries no value: weights e^{s_t} / (1 + sum e^{s_t}).  Values may have a width
// of their own (-DLLB_VALUE_DIM, default the head size).  `sink_logits` gives the sink a learned score per query
// head instead of 0 (the term e^{sink_h}).  With `v_in_k` the values are the leading LLB_VALUE_DIM elements of the key
// rows themselves (a cache of one latent row per token that serves as key and as value; no value pool is read).
// `kv_row_stride` > 0: the step's own keys (and values) stand in a buffer of their own with that row stride.
// `dist_r1`, `dist_r2` (two numbers per query head): a score loses r1 ln(1 + r2 (p - t)), a penalty that grows with the
// distance.  `q_temp_every` > 0: the query at position p is multiplied by 1 + q_temp_coef ln(floor((p + 1) / every) + 1).
// `chunk` C > 0: the query at position p sees no key before floor(p / C) * C.  `maps` M > 1: M key heads share one value
// head (several score maps over one set of values) and a cache key row holds their keys side by side.  `pool` P > 0 (with a
// window W): beside the window's keys, one key and value per block of P positions that lies wholly before the window
// (block b is seen from p when b P + P - 1 <= p - W), read at row b of a second cache and walked before the window's tiles;
// tokens and blocks share one softmax.  `out_f32`: the result is float32 whatever the operands are.
//
// Keys are walked in tiles of one cache page with an online softmax, so nothing of size
// [queries, keys] is ever stored.
//
//  * prefill: a block owns 32 consecutive new tokens of one head of one sequence.  Keys at
//    positions before the step come from the cache pages, keys of the step itself from the
//    packed projection output (the cache is appended to afterwards, which lets a window layer
//    keep a ring of pages shorter than the prompt).
//  * decode: one new token per sequence, already appended.  A block owns the query heads that
//    share one kv head and one slice of the key range; slices are merged by llb_attn_combine.
#include "common.cuh"

#ifndef LLB_HEAD_DIM
#error "compile with -DLLB_HEAD_DIM=<head size>"
#endif

#ifndef LLB_VALUE_DIM
#define LLB_VALUE_DIM LLB_HEAD_DIM
#endif

constexpr int DH = LLB_HEAD_DIM;     // query / key width
constexpr int DV = LLB_VALUE_DIM;    // value and output width
// query rows of a block: 32, or 8 for keys so wide that 32 rows and a key tile no longer fit an SM's shared memory
constexpr bool ROWS32_FIT = (size_t)(32 * DH + LLB_PAGE * (DH + 1) + 4 * LLB_PAGE) * sizeof(float) <= 227 * 1024;
constexpr int ROWS = (DH <= 256 || ROWS32_FIT) ? 32 : 8;
constexpr int WARPS = 4;
constexpr int RPW = ROWS / WARPS;   // rows of a warp
constexpr int DPL = (DV + 31) / 32; // output dims of a lane

struct AttnParams {
    const void* q;        // packed projections [T, row_stride]; query head h at column h * DH
    const void* k_new;    // the same buffer at its first key column
    const void* v_new;    // the same buffer at its first value column
    int row_stride;
    void* out;            // [T, nh * DV]
    const void* kpool;    // [pages, nkvh, LLB_PAGE, DH]
    const void* vpool;    // [pages, nkvh, LLB_PAGE, DV]
    const int* page_table;  // [B, table_stride]
    int table_stride;
    int ring;
    const int* seq_start;       // [B + 1] first packed token of each sequence
    const int* seq_len_before;  // [B] tokens in the cache before this step
    int nh, nkvh, window;
    float scale;
    int all_from_cache;   // prefill only: the step's own keys are already in the cache (a call that
                          // reads another call's cache); read nothing from k_new / v_new
    int n_splits;         // decode only
    float* part_o;        // decode only: [B, nh, n_splits, DV]
    float* part_ml;       // decode only: [B, nh, n_splits, 2]
    int keep_first;       // with a window: keys before this position stay visible
    int pinned;           // pages ahead of the ring that are never overwritten
    int sink;             // the softmax's denominator has one more term e^0
    const float* sink_logits;   // [nh] or null: the sink's score per query head instead of 0 (implies a sink)
    int v_in_k;           // values are the first DV elements of the key rows; vpool and v_new are not read
    int kv_row_stride;    // row stride of k_new / v_new when they are no part of the q buffer (0: row_stride)
    const float* dist_r1; // [nh] or null: a score loses dist_r1[h] * ln(1 + dist_r2[h] * (query position - key position))
    const float* dist_r2;
    float q_temp_coef;    // with q_temp_every > 0 the query at position p is multiplied by
    int q_temp_every;     //   1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1)
    int chunk;            // > 0: a query at position p sees no key before floor(p / chunk) * chunk
    int maps;             // > 1: `maps` key heads share one value head; nkvh counts key heads, the cache has nkvh / maps
                          //      heads whose key rows hold the maps' keys side by side (maps * DH elements)
    int out_f32;          // out is float32 whatever the operands' type
    int pool;             // > 0 (with a window): beside the window's keys, one key and value per block of `pool` positions
                          //      that lies wholly before the window (block b: b * pool + pool - 1 <= p - window), read
                          //      at row b of a second cache; tokens and blocks share one softmax
    const void* pool_k;   // [pages, nkvh / maps, LLB_PAGE, maps * DH]
    const void* pool_v;   // [pages, nkvh / maps, LLB_PAGE, DV]
    const int* pool_table;  // [B, pool_table_stride]
    int pool_table_stride;
};

template <typename T, bool DECODE>
__global__ void __launch_bounds__(WARPS * 32) attn_kernel(AttnParams p) {
    extern __shared__ float smem[];
    float* Qs = smem;                        // [ROWS][DH]
    float* Ks = Qs + ROWS * DH;              // [LLB_PAGE][DH + 1]
    float* Vs = Ks + LLB_PAGE * (DH + 1);    // [LLB_PAGE][DV]; with v_in_k the key tile itself
    float* Ps = Vs + (p.v_in_k ? 0 : LLB_PAGE * DV);   // [WARPS][LLB_PAGE]
    const int vs_stride = p.v_in_k ? DH + 1 : DV;
    if (p.v_in_k) Vs = Ks;
    const int kv_stride = p.kv_row_stride > 0 ? p.kv_row_stride : p.row_stride;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.z;
    llb_grid_dependency_sync();
    const int tok0 = p.seq_start[b];
    const int n_new = p.seq_start[b + 1] - tok0;
    const int len_before = p.seq_len_before[b];
    const int G = p.nh / p.nkvh;
    const int maps = p.maps > 1 ? p.maps : 1, cache_heads = p.nkvh / maps, krow = DH * maps;
    const int* table = p.page_table + (size_t)b * p.table_stride;

    // ---- the rows of this block: (token, head, position) per row
    int kvh, n_rows, first_pos, last_pos;
    int row_tok0, row_head0;                 // row r: token row_tok0 + (DECODE ? 0 : r), head row_head0 + (DECODE ? r : 0)
    if (DECODE) {
        int chunks = (G + ROWS - 1) / ROWS;
        kvh = blockIdx.y / chunks;
        int c = blockIdx.y - kvh * chunks;
        n_rows = min(ROWS, G - c * ROWS);
        row_head0 = kvh * G + c * ROWS;
        row_tok0 = tok0;
        first_pos = last_pos = len_before;   // n_new == 1
    } else {
        int t0 = blockIdx.x * ROWS;
        if (t0 >= n_new) return;
        n_rows = min(ROWS, n_new - t0);
        row_head0 = blockIdx.y;
        kvh = row_head0 / G;
        row_tok0 = tok0 + t0;
        first_pos = len_before + t0;
        last_pos = first_pos + n_rows - 1;
    }
    const int vh = kvh / maps, kmap = kvh - vh * maps;     // the key head's value head and its place in the cache's key row
    const T* qbase = (const T*)p.q;
    for (int i = tid; i < n_rows * DH; i += WARPS * 32) {
        int r = i / DH, d = i - r * DH;
        int tok = row_tok0 + (DECODE ? 0 : r), head = row_head0 + (DECODE ? r : 0);
        Qs[r * DH + d] = to_f32(qbase[(size_t)tok * p.row_stride + head * DH + d]);
    }

    // ---- key tiles of this block: the tiles of the kept first keys that lie before the window's, then the window's
    const int keep = p.window > 0 ? p.keep_first : 0;
    int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    if (p.chunk > 0) key_lo = max(key_lo, (first_pos / p.chunk) * p.chunk);
    const int tile_lo = key_lo / LLB_PAGE, tile_hi = last_pos / LLB_PAGE + 1;
    const int n_kept = min((keep + LLB_PAGE - 1) / LLB_PAGE, tile_lo);
    // pooled blocks that the block's last row sees, and their tiles (walked first)
    const int blocks_hi = (p.pool > 0 && p.window > 0) ? max(0, (last_pos - p.window + 1) / p.pool) : 0;
    const int n_pool = (blocks_hi + LLB_PAGE - 1) / LLB_PAGE;
    int it_lo = 0, it_hi = n_pool + n_kept + tile_hi - tile_lo;   // after the pooled tiles: it < n_kept ? it : tile_lo + it - n_kept
    if (DECODE) {
        int chunk = (it_hi + p.n_splits - 1) / p.n_splits;
        it_lo = blockIdx.x * chunk;
        it_hi = min(it_hi, it_lo + chunk);
    }
    const bool with_sink = (p.sink || p.sink_logits) && (!DECODE || blockIdx.x == 0);

    float m[RPW], l[RPW], o[RPW][DPL];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp + i * WARPS;
        m[i] = with_sink ? (p.sink_logits ? p.sink_logits[row_head0 + (DECODE ? min(r, n_rows - 1) : 0)] : 0.f) : -INFINITY;
        l[i] = with_sink ? 1.f : 0.f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) o[i][e] = 0.f;
    }

    const T* kpool = (const T*)p.kpool;
    const T* vpool = (const T*)p.vpool;
    const T* knew = (const T*)p.k_new;
    const T* vnew = (const T*)p.v_new;

    for (int it = it_lo; it < it_hi; ++it) {
        const bool pooled = it < n_pool;
        const int tile = pooled ? it : (it - n_pool < n_kept ? it - n_pool : tile_lo + it - n_pool - n_kept);
        __syncthreads();                     // previous tile fully consumed (and Qs written)
        // A tile is one cache page (tiles start at multiples of LLB_PAGE): its page is looked up once; rows move in
        // 16-byte pieces where the widths and the addresses allow it.
        const int p0 = tile * LLB_PAGE;
        // (the page table is read only for a tile that holds cached positions: a step without history may come with
        // an empty table)
        if (pooled) {
            const int* ptab = p.pool_table + (size_t)b * p.pool_table_stride;
            const T* kp = (const T*)p.pool_k + paged_row(ptab, p.pool_table_stride, p0, vh, cache_heads, krow, 0) + kmap * DH;
            const T* vp = (const T*)p.pool_v + paged_row(ptab, p.pool_table_stride, p0, vh, cache_heads, DV, 0);
            for (int i = tid; i < LLB_PAGE * DH; i += WARPS * 32) {
                const int j = i / DH, d = i - j * DH;
                Ks[j * (DH + 1) + d] = p0 + j < blocks_hi ? to_f32(kp[(size_t)j * krow + d]) : 0.f;
            }
            for (int i = tid; i < LLB_PAGE * DV; i += WARPS * 32) {
                const int j = i / DV, d = i - j * DV;
                Vs[j * DV + d] = p0 + j < blocks_hi ? to_f32(vp[(size_t)j * DV + d]) : 0.f;
            }
        }
        const bool cached = DECODE || p.all_from_cache || p0 < len_before;
        const T* kpage = (cached && !pooled) ? kpool + paged_row(table, p.ring, p0, vh, cache_heads, krow, p.pinned) + kmap * DH : nullptr;
        constexpr int VEC = 16 / (int)sizeof(T);
        const bool kvec = DH % VEC == 0 && (((uintptr_t)kpool | (uintptr_t)knew) & 15) == 0 && kv_stride % VEC == 0;
        if (pooled) {
        } else if (kvec) {
            // eight pieces a thread are requested before the first is used: the walk waits for memory once per batch
            constexpr int PIECES = LLB_PAGE * (DH / VEC), BATCH = 8;
            for (int i0 = tid; i0 < PIECES; i0 += BATCH * WARPS * 32) {
                uint4 raw[BATCH];
#pragma unroll
                for (int u = 0; u < BATCH; ++u) {
                    const int i = i0 + u * WARPS * 32;
                    raw[u] = make_uint4(0u, 0u, 0u, 0u);                 // zero bits are zero in both types
                    if (i < PIECES) {
                        const int j = i / (DH / VEC), d = (i - j * (DH / VEC)) * VEC, kp = p0 + j;
                        if ((kp >= key_lo || kp < keep) && kp <= last_pos) {
                            const T* src = (!DECODE && !p.all_from_cache && kp >= len_before)
                                               ? knew + (size_t)(tok0 + kp - len_before) * kv_stride + kvh * DH + d
                                               : kpage + (size_t)j * krow + d;
                            raw[u] = *reinterpret_cast<const uint4*>(src);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < BATCH; ++u) {
                    const int i = i0 + u * WARPS * 32;
                    if (i < PIECES) {
                        const int j = i / (DH / VEC), d = (i - j * (DH / VEC)) * VEC;
                        const T* rv = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) Ks[j * (DH + 1) + d + e] = to_f32(rv[e]);
                    }
                }
            }
        } else {
            for (int i = tid; i < LLB_PAGE * DH; i += WARPS * 32) {
                int j = i / DH, d = i - j * DH;
                int kp = p0 + j;
                float kv = 0.f;
                if ((kp >= key_lo || kp < keep) && kp <= last_pos) {
                    if (!DECODE && !p.all_from_cache && kp >= len_before)
                        kv = to_f32(knew[(size_t)(tok0 + kp - len_before) * kv_stride + kvh * DH + d]);
                    else
                        kv = to_f32(kpage[(size_t)j * krow + d]);
                }
                Ks[j * (DH + 1) + d] = kv;
            }
        }
        if (!p.v_in_k && !pooled) {
            const T* vpage = cached ? vpool + paged_row(table, p.ring, p0, vh, cache_heads, DV, p.pinned) : nullptr;
            for (int i = tid; i < LLB_PAGE * DV; i += WARPS * 32) {
                int j = i / DV, d = i - j * DV;
                int kp = p0 + j;
                float vv = 0.f;
                if ((kp >= key_lo || kp < keep) && kp <= last_pos) {
                    if (!DECODE && !p.all_from_cache && kp >= len_before)
                        vv = to_f32(vnew[(size_t)(tok0 + kp - len_before) * kv_stride + vh * DV + d]);
                    else
                        vv = to_f32(vpage[(size_t)j * DV + d]);
                }
                Vs[j * DV + d] = vv;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            int r = warp + i * WARPS;
            if (r >= n_rows) continue;       // uniform within the warp
            int pos = DECODE ? first_pos : first_pos + r;
            int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            if (p.chunk > 0) lo = max(lo, (pos / p.chunk) * p.chunk);
            const int blocks_seen = pooled ? max(0, (pos - p.window + 1) / p.pool) : 0;
            float row_scale = p.scale;
            if (p.q_temp_every > 0) row_scale *= 1.0f + p.q_temp_coef * logf((float)((pos + 1) / p.q_temp_every + 1));
            float r1 = 0.f, r2 = 0.f;
            if (p.dist_r1) {
                const int head = row_head0 + (DECODE ? r : 0);
                r1 = p.dist_r1[head];
                r2 = p.dist_r2[head];
            }
            const float* qr = Qs + r * DH;
            const float* k0 = Ks + lane * (DH + 1);
            const float* k1 = Ks + (lane + 32) * (DH + 1);
            // four partial sums a key: eight independent chains, so that a product does not wait for the one before it
            // (with one chain a key the warp spent most cycles on the latency of its own additions)
            float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                int d = 0;
#pragma unroll 4
                for (; d + 4 <= DH; d += 4) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float qv = qr[d + u];
                        a0[u] = fmaf(qv, k0[d + u], a0[u]);
                        a1[u] = fmaf(qv, k1[d + u], a1[u]);
                    }
                }
                for (; d < DH; ++d) {
                    a0[0] = fmaf(qr[d], k0[d], a0[0]);
                    a1[0] = fmaf(qr[d], k1[d], a1[0]);
                }
            }
            float s0 = (a0[0] + a0[1]) + (a0[2] + a0[3]), s1 = (a1[0] + a1[1]) + (a1[2] + a1[3]);
            int kp0 = tile * LLB_PAGE + lane, kp1 = kp0 + 32;
            bool v0 = (kp0 >= lo || kp0 < keep) && kp0 <= pos, v1 = (kp1 >= lo || kp1 < keep) && kp1 <= pos;
            if (pooled) {
                v0 = kp0 < blocks_seen;
                v1 = kp1 < blocks_seen;
            }
            s0 = v0 ? s0 * row_scale : -INFINITY;
            s1 = v1 ? s1 * row_scale : -INFINITY;
            if (p.dist_r1 && !pooled) {
                if (v0) s0 -= r1 * log1pf(r2 * (float)(pos - kp0));
                if (v1) s1 -= r1 * log1pf(r2 * (float)(pos - kp1));
            }
            float m_new = fmaxf(m[i], warp_max(fmaxf(s0, s1)));
            if (m_new == -INFINITY) continue;          // no visible key yet (uniform)
            float alpha = expf(m[i] - m_new);           // exp(-inf) = 0 on the first visible tile
            float p0 = v0 ? expf(s0 - m_new) : 0.f, p1 = v1 ? expf(s1 - m_new) : 0.f;
            l[i] = l[i] * alpha + warp_sum(p0 + p1);
            m[i] = m_new;
            float* ps = Ps + warp * LLB_PAGE;
            __syncwarp();
            ps[lane] = p0;
            ps[lane + 32] = p1;
            __syncwarp();
            // keys outside, the lane's output dimensions inside: DPL independent chains
#pragma unroll
            for (int e = 0; e < DPL; ++e) o[i][e] *= alpha;
#pragma unroll 4
            for (int j = 0; j < LLB_PAGE; ++j) {
                const float pj = ps[j];
                const float* vr = Vs + j * vs_stride + lane;
#pragma unroll
                for (int e = 0; e < DPL; ++e)
                    if (lane + e * 32 < DV) o[i][e] = fmaf(pj, vr[e * 32], o[i][e]);
            }
        }
    }

    // ---- write out
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        int r = warp + i * WARPS;
        if (r >= n_rows) continue;
        int tok = row_tok0 + (DECODE ? 0 : r), head = row_head0 + (DECODE ? r : 0);
        if (!DECODE || p.n_splits == 1) {
            const size_t at = (size_t)tok * p.nh * DV + head * DV;
            float inv = 1.0f / l[i];
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int d = lane + e * 32;
                if (d < DV) {
                    if (p.out_f32) ((float*)p.out)[at + d] = o[i][e] * inv;
                    else ((T*)p.out)[at + d] = from_f32<T>(o[i][e] * inv);
                }
            }
        } else {
            size_t slot = ((size_t)b * p.nh + head) * p.n_splits + blockIdx.x;
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int d = lane + e * 32;
                if (d < DV) p.part_o[slot * DV + d] = o[i][e];
            }
            if (lane == 0) {
                p.part_ml[slot * 2] = m[i];
                p.part_ml[slot * 2 + 1] = l[i];
            }
        }
    }
}

// Merges the key slices of decode: out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M).
template <typename T>
__global__ void attn_combine_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, const int* __restrict__ seq_start,
                                    int nh, int n_splits) {
    llb_grid_dependency_sync();
    int head = blockIdx.x, b = blockIdx.y;
    size_t base = ((size_t)b * nh + head) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        float ms = part_ml[(base + s) * 2];
        if (ms != -INFINITY) L += part_ml[(base + s) * 2 + 1] * expf(ms - M);
    }
    int tok = seq_start[b];
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ms = part_ml[(base + s) * 2];
            if (ms != -INFINITY) acc += part_o[(base + s) * DV + d] * expf(ms - M);
        }
        out[(size_t)tok * nh * DV + head * DV + d] = from_f32<T>(acc / L);
    }
}

static size_t attn_smem_bytes(bool v_in_k) {
    return (size_t)(ROWS * DH + LLB_PAGE * (DH + 1) + (v_in_k ? 0 : LLB_PAGE * DV) + WARPS * LLB_PAGE) * sizeof(float);
}

template <typename T, bool DECODE>
static int launch_attn(const AttnParams& p, dim3 grid, cudaStream_t stream) {
    auto k = attn_kernel<T, DECODE>;
    size_t smem = attn_smem_bytes(p.v_in_k != 0);
    static bool configured = false;          // once per instantiation: not repeated inside a graph capture
    if (!configured && attn_smem_bytes(false) > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(p.v_in_k && attn_smem_bytes(false) > 227 * 1024 ? smem : attn_smem_bytes(false)));
        if (e != cudaSuccess) return (int)e;
    }
    configured = true;
    llb_launch(k, grid, dim3(WARPS * 32), smem, stream, p);
    return llb_status();
}

// Prefill and any step with more than one new token in some sequence.  max_new is the largest
// number of new tokens of a sequence in the batch.
LLB_API int llb_attn_prefill(AttnParams p, int dtype, int B, int max_new, cudaStream_t stream) {
    if (B == 0 || max_new == 0) return 0;
    if (p.nkvh <= 0 || p.nh % p.nkvh || (p.maps > 1 && p.nkvh % p.maps)) return (int)cudaErrorInvalidValue;
    dim3 grid((max_new + ROWS - 1) / ROWS, p.nh, B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, T, return launch_attn<T, false>(p, grid, stream));
    return 0;
}

// Decode: every sequence has exactly one new token, already in the cache.
LLB_API int llb_attn_decode(AttnParams p, int dtype, int B, cudaStream_t stream) {
    if (B == 0) return 0;
    if (p.nkvh <= 0 || p.nh % p.nkvh || p.n_splits < 1 || (p.maps > 1 && p.nkvh % p.maps)) return (int)cudaErrorInvalidValue;
    int G = p.nh / p.nkvh;
    dim3 grid(p.n_splits, p.nkvh * ((G + ROWS - 1) / ROWS), B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    int rc;
    LLB_DISPATCH_DTYPE(dtype, T, {
        rc = launch_attn<T, true>(p, grid, stream);
        if (rc == 0 && p.n_splits > 1) {
            if (p.out_f32)
                llb_launch(attn_combine_kernel<float>, dim3(p.nh, B), dim3(128), 0, stream,
                           (float*)p.out, (const float*)p.part_o, (const float*)p.part_ml, p.seq_start, p.nh, p.n_splits);
            else
                llb_launch(attn_combine_kernel<T>, dim3(p.nh, B), dim3(128), 0, stream,
                           (T*)p.out, (const float*)p.part_o, (const float*)p.part_ml, p.seq_start, p.nh, p.n_splits);
            rc = llb_status();
        }
        return rc;
    });
    return 0;
}
