// The experts' matrix products on the 5th-generation tensor cores (tcgen05), bfloat16 operands, float32 accumulation.
//
// A step's (token, choice) pairs are grouped by expert and cut into tiles of BN slots (csrc/moe.cu, the plan; BN is 16,
// 64 or 128, chosen by how many pairs an expert gets on average).  A block owns one tile and 128 consecutive rows of
// that tile's expert matrix: the weight rows are the UMMA's M operand, the tile's slots its N operand, both K-major,
// as in csrc/gemm_tc.cu.  The experts' matrices lie
// stacked as one [E * N, K] matrix, so one tensor map serves all experts and a block finds its rows at
// expert * N + row block; the activations lie in slot order ([slots, K]: gathered rows of the step's tokens for the up
// projection, the up projection's own output for the down projection), so a tile's operand is one box at its first
// slot.  What a box holds beyond the expert's rows or the tile's slots (the next expert's, or zeros outside the
// matrices) is computed and not stored.
//
//   TMA (128-byte swizzle) -> ring of STAGES k-blocks -> tcgen05.mma by one elected lane, accumulator in tensor memory
//   -> tcgen05.ld by four warps -> the epilogue:
//        store         out[slot, n] = act(acc)                     (act: none, max(., 0)^2 or gelu, erf form)
//        weighted add  stream[token(slot), n] += weight(slot) * acc   (float32 atomics: a token's chosen experts and
//                      the layer's other branches meet in the stream in arrival order)
//
// The grid covers the most tiles the step's shape allows; blocks beyond the step's real number of tiles (known on the
// device only) leave at once.  Every mbarrier wait is bounded (errors 151-153): the block records the code, waits
// (bounded) for its copies in flight, frees its tensor memory and returns.
#include "common.cuh"
#include "tma_map.cuh"
#include "umma.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int A_BYTES = BM * BK * 2;
template <int BN, int STAGES>
struct Shape {                          // two blocks share an SM: under 113 KB each
    static constexpr int B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int SMEM_TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
};
enum { ERR_MOE_WAIT_FULL = 151, ERR_MOE_WAIT_EMPTY = 152, ERR_MOE_WAIT_ACC = 153 };
enum { EPI_STORE = 0, EPI_RELU2 = 1, EPI_WEIGHTED_ADD = 2, EPI_GELU = 3 };

struct MoeTcArgs {
    void* out;                 // store: [slots, ldo] bfloat16 or float32; weighted add: the float32 stream [T, ldo]
    int out_dtype, ldo;
    const int* tiles;          // [3, max_tiles]: expert, first slot, rows
    int max_tiles;
    const int* n_tiles;
    int N, K, epilogue;
    const int* pair_of;        // weighted add: slot -> pair (token * top + choice)
    const float* wgt;          //               pair -> weight
    int top;
    int* err;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, MoeTcArgs g) {
    using S = Shape<BN, STAGES>;
    constexpr int STAGE_BYTES = S::STAGE_BYTES, BAR_OFFSET = S::BAR_OFFSET, TMEM_COLS = S::TMEM_COLS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_full = base + BAR_OFFSET, bar_empty = bar_full + 8 * STAGES, bar_acc = bar_empty + 8 * STAGES;
    const uint32_t tmem_slot = bar_acc + 8;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + BAR_OFFSET + (2 * STAGES + 1) * 8);
    __shared__ int s_abort;
    static_assert(BN <= THREADS, "a thread per slot fills the tile's tokens and weights");
    __shared__ int s_token[BN];
    __shared__ float s_weight[BN];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;

    llb_grid_dependency_sync();          // the plan (and the activations) come from kernels of this step
    const int tile = blockIdx.y;
    const bool active = tile < *g.n_tiles;                     // the same for every thread of the block
    if (active) {
        const int e = g.tiles[tile], slot0 = g.tiles[g.max_tiles + tile], rows = g.tiles[2 * g.max_tiles + tile];
        const int m0 = blockIdx.x * BM;
        const int kblocks = (g.K + BK - 1) / BK;
        if (g.epilogue == EPI_WEIGHTED_ADD && tid < BN) {
            const int pair = tid < rows ? g.pair_of[slot0 + tid] : 0;
            s_token[tid] = pair / g.top;
            s_weight[tid] = tid < rows ? g.wgt[pair] : 0.f;
        }
        if (warp == 0) {
            if (lane == 0) {
                // ---- producer: whole k-blocks (128 weight rows, 64 slots) into the ring
                int issued = 0;
                for (int kb = 0; kb < kblocks; ++kb, ++issued) {
                    const int s = issued % STAGES;
                    const uint32_t round = issued / STAGES;
                    if (round > 0 && !mbar_wait(bar_empty + 8 * s, (round - 1) & 1, &s_abort)) {
                        if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_MOE_WAIT_EMPTY); }
                        break;
                    }
                    const uint32_t dst = base + s * STAGE_BYTES;
                    mbar_expect_tx(bar_full + 8 * s, STAGE_BYTES);
                    // few slots per expert (decode): a weight tile is read once; many (prefill): the expert's next tiles read it again
                    tma_load_2d(dst, &map_w, bar_full + 8 * s, kb * BK, e * g.N + m0, BN <= 16 ? HINT_EVICT_FIRST : HINT_EVICT_LAST);
                    tma_load_2d(dst + A_BYTES, &map_x, bar_full + 8 * s, kb * BK, slot0, HINT_EVICT_LAST);
                }
                if (s_abort) {
                    // copies in flight must land before this block's shared memory is given up
                    const int first = issued > STAGES ? issued - STAGES : 0;
                    for (int i = first; i < issued; ++i)
                        for (uint32_t t = 0; t < WAIT_LIMIT && !mbar_try(bar_full + 8 * (i % STAGES), (i / STAGES) & 1); ++t) {}
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // ---- tensor-core issue: the warp waits as a whole, one elected lane issues
            const uint32_t idesc = umma_idesc(BN);
            const uint64_t a_desc0 = umma_desc(base), b_desc0 = umma_desc(base + A_BYTES);
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < kblocks; ++kb) {
                if (!warp_wait(bar_full + 8 * s, ph, &s_abort)) {
                    if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MOE_WAIT_FULL); }
                    break;
                }
                if (elect_one()) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t so = (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t off = so + (uint64_t)((k * UMMA_K * 2) >> 4);
                        umma(tmem, a_desc0 + off, b_desc0 + off, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * s);       // the stage is free once these products have read it
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
            if (elect_one()) umma_commit(bar_acc);        // accumulator complete (arrives even after an early stop)
            __syncwarp();
        }

        // ---- epilogue: warp w owns tensor-memory lanes 32 w .. 32 w + 31 = weight rows (output columns) m0 + 32 w ..
        const bool ok = mbar_wait(bar_acc, 0, &s_abort);
        if (!ok && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MOE_WAIT_ACC); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        __syncthreads();
        if (!s_abort) {
            const int n = m0 + tid;
            const bool col_ok = n < g.N;
            const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (c >= rows) break;                      // (the same for every thread)
                float v[16];
                tmem_ld16(lane_addr + c, v);               // warp-collective
                if (!col_ok) continue;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c + j >= rows) break;
                    float x = v[j];
                    if (g.epilogue == EPI_WEIGHTED_ADD) {
                        atomicAdd((float*)g.out + (size_t)s_token[c + j] * g.ldo + n, s_weight[c + j] * x);
                        continue;
                    }
                    if (g.epilogue == EPI_RELU2) {
                        x = fmaxf(x, 0.f);
                        x *= x;
                    }
                    if (g.epilogue == EPI_GELU) x = 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
                    const size_t o = (size_t)(slot0 + c + j) * g.ldo + n;
                    if (g.out_dtype == LLB_F32) ((float*)g.out)[o] = x;
                    else ((bf16*)g.out)[o] = __float2bfloat16_rn(x);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

}  // namespace

template <int BN, int STAGES>
static int launch_moe_tc(const CUtensorMap& mw, const CUtensorMap& mx, const MoeTcArgs& g, dim3 grid, cudaStream_t stream) {
    auto k = moe_gemm_tc_kernel<BN, STAGES>;
    constexpr int smem = Shape<BN, STAGES>::SMEM_TOTAL;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return -2000 - (int)e;
        configured[dev] = true;
    }
    llb_launch(k, grid, dim3(THREADS), (size_t)smem, stream, mw, mx, g);
    return llb_status();
}

// A [slots, K] bfloat16 (row stride lda) in slot order; W [E, N, K] bfloat16, dense; tiles of tile_rows (16, 64 or 128)
// slots as the plan cut them.  epilogue 0: out[slots, ldo] = product; 1: its squared ReLU; 3: its gelu (erf form); 2: out is the float32 stream
// [T, ldo] and row token(slot) gets weight(slot) * product added.  K must be a multiple of 8 and all bases 16-byte aligned.
LLB_API int llb_moe_gemm_tc(const void* A, int lda, long long n_slots, const void* W, int E, int N, int K, void* out, int out_dtype,
                            int ldo, const int* tiles, int max_tiles, const int* n_tiles, int tile_rows, int epilogue,
                            const int* pair_of, const float* wgt, int top, int* err, cudaStream_t stream) {
    const int BN = tile_rows;
    if (BN != 16 && BN != 64 && BN != 128) return (int)cudaErrorInvalidValue;
    if (max_tiles == 0 || N == 0 || n_slots == 0) return 0;
    if (K % 8 || lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || epilogue < 0 || epilogue > 3) return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_WEIGHTED_ADD && (!pair_of || !wgt || top < 1 || out_dtype != LLB_F32)) return (int)cudaErrorInvalidValue;
    if (out_dtype != LLB_F32 && out_dtype != LLB_BF16) return (int)cudaErrorInvalidValue;
    dim3 grid((N + BM - 1) / BM, max_tiles);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    CUtensorMap mw, mx;
    int rc = llb_tma::bf16_map_64(W, (long long)E * N, K, K, BM, &mw);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(A, n_slots, K, lda, BN, &mx);
    if (rc) return rc;
    MoeTcArgs g{out, out_dtype, ldo, tiles, max_tiles, n_tiles, N, K, epilogue, pair_of, wgt, top, err};
    // (Measured at 2,048 tokens, 64 experts of 1,536 x 4,096, 8 per token: six stages with one block per SM instead of
    // three with two took 441 us instead of 307; the product is bound by what 128 x 128 tiles pull from L2, not by latency.)
    switch (BN) {
        case 16: return launch_moe_tc<16, 5>(mw, mx, g, grid, stream);        //  91 KB
        case 64: return launch_moe_tc<64, 4>(mw, mx, g, grid, stream);        //  97 KB
        default: return launch_moe_tc<128, 3>(mw, mx, g, grid, stream);       //  97 KB
    }
}
