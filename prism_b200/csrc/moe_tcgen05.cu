// The experts' grouped products on the 5th-generation tensor cores (bf16 operands, float32 accumulation).
//
// The (token, choice) rows are sorted by expert, every expert's stretch starting at a multiple of the token tile
// (prism_moe_place with pad = the tile), so that a tile of NTOK rows belongs to one expert.  As in the weight-
// streaming product (gemm_tcgen05.cu) the roles are swapped: 128 rows of the expert's matrix are the M dimension of
// one tcgen05.mma and the tile's rows its N dimension, TMA brings both through a ring of shared-memory stages, one
// thread issues the MMAs into tensor memory, four warps read the accumulator back.
//
//   grid (tiles of 128 output features of ONE expert, token tiles): CTA (i, j) looks up the expert e of token tile j
//   in the padded offsets (after pdl_wait: the kernel before wrote them), leaves if the tile lies beyond the last
//   stretch, and loads the rows  e rows_per_expert + 128 i ..  of the weight matrix, seen as [E rows_per_expert, K].
//   Rows of the tile past the expert's own (the next matrix's, or none) feed accumulator lanes that are not stored.
//
//   dual:   hidden[p, n] = act(gate_e a_p)[n] * (up_e a_p)[n]   bf16, p the padded row; W is [E, 2 N, K]
//   single: y[dst[p], n] = (down_e h_p)[n] (* weight[p])         float32; W is [E, N, K]
//           without dst: hidden[p, n] = act(up_e a_p)[n]         bf16: the hidden layer of experts without a gate
//
// A decode step (a few rows per expert) reads every chosen expert's weights once; a prompt's tiles of one expert
// re-read them from L2.  Every mbarrier wait is bounded, as in gemm_tcgen05.cu.
#include "tcgen05.cuh"

namespace prism {
namespace tc {

constexpr int MOE_TILE_M = 128;
constexpr int MOE_THREADS = 192;

__device__ __forceinline__ float moe_tc_act(float z, int act) {
    if (act == 0) return z / (1.f + expf(-z));                                                      // silu
    if (act == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));   // gelu_tanh
    const float r = fmaxf(z, 0.f);
    return act == 3 ? r * r : r;                                                                      // relu squared, relu
}

template <int NTOK, bool DUAL> struct MoeCfg {
    static constexpr int W_TILES = DUAL ? 2 : 1;
    static constexpr int STAGE_BYTES = W_TILES * MOE_TILE_M * TILE_K * 2 + NTOK * TILE_K * 2;
    // the down product of a prompt's tiles (K = an expert's inner width: few k-blocks, 64 rows to scatter): a short ring,
    // so that three CTAs share an SM and one's store hides behind the others' products; decode steps stream weights
    // and keep the deep ring
    static constexpr int FIT = ((DUAL || NTOK < 64) ? 200 : 72) * 1024 / STAGE_BYTES;
    static constexpr int STAGES = FIT >= 6 ? 6 : (FIT >= 2 ? FIT : 2);
    static constexpr int TMEM_COLS = (W_TILES * NTOK) <= 32 ? 32 : ((W_TILES * NTOK) <= 64 ? 64 : 128);
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
};

template <int NTOK, bool DUAL>
__global__ void __launch_bounds__(MOE_THREADS)
moe_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const int* __restrict__ offs_in, const int* __restrict__ counts_in, const int* __restrict__ row_dst_in,
                const float* __restrict__ row_w_in, int E, int N, int K, int act, void* __restrict__ y, long long ldy,
                int* err) {
    using C = MoeCfg<NTOK, DUAL>;
    constexpr int W_TILES = C::W_TILES;
    constexpr int STAGES = C::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    __shared__ int abort_flag;
    __shared__ int tile_e, tile_valid;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.y * NTOK;                    // first padded row of this token tile
    pdl_trigger();
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_wait();
        const int* offs = pdl_fresh(offs_in);
        const int* counts = pdl_fresh(counts_in);
        int found = -1, valid = 0;
        for (int e = 0; e < E; ++e) {
            const int a = offs[e], b = offs[e + 1];
            if (row0 >= a && row0 < b) {
                found = e;
                valid = min(NTOK, a + counts[e] - row0);
                break;
            }
        }
        tile_e = found;
        tile_valid = valid;
    }
    __syncthreads();
    const int e = tile_e, valid = tile_valid;
    if (e < 0 || valid <= 0) return;                       // the whole CTA: nothing allocated yet
    const int m_in = blockIdx.x * MOE_TILE_M;              // first output feature of this tile, inside the expert
    const int w_row0 = e * (DUAL ? 2 : 1) * N + m_in;
    const int nkb = (K + TILE_K - 1) / TILE_K;

    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(C::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    volatile int* abortp = &abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            int issued = 0;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abortp)) break;
                unsigned char* st = tiles + (size_t)s * C::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                const int kc = i * TILE_K;
#pragma unroll
                for (int w = 0; w < W_TILES; ++w)
                    tma_load_2d(st + w * MOE_TILE_M * TILE_K * 2, &map_w, &full_bar[s], kc, w_row0 + w * N);
                tma_load_2d(st + W_TILES * MOE_TILE_M * TILE_K * 2, &map_x, &full_bar[s], kc, row0);
                issued = i + 1;
            }
            if (*abortp) {
                for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1, abortp);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) |
                                       ((uint32_t)(MOE_TILE_M >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&full_bar[s], (i / STAGES) & 1, abortp);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t st = smem_addr(tiles + (size_t)s * C::STAGE_BYTES);
                const uint64_t db = umma_desc(st + W_TILES * MOE_TILE_M * TILE_K * 2);
#pragma unroll
                for (int w = 0; w < W_TILES; ++w) {
                    const uint64_t da = umma_desc(st + w * MOE_TILE_M * TILE_K * 2);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        umma_bf16(tmem_base + w * NTOK, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4),
                                  idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);
            }
            umma_commit(acc_bar);
        }
    } else {
        const int q = warp & 3;
        const int m = m_in + q * 32 + lane;              // this thread's output feature inside the expert
        pdl_wait();
        const int* row_dst = pdl_fresh(row_dst_in);
        const float* row_w = pdl_fresh(row_w_in);
        mbar_wait(acc_bar, 0, abortp);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool go = *abortp == 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (go) {
            float acc[W_TILES][NTOK];
#pragma unroll
            for (int w = 0; w < W_TILES; ++w) tmem_load<NTOK>(tmem_base + ((uint32_t)(q * 32) << 16) + w * NTOK, acc[w]);
            if (m < N) {
#pragma unroll
                for (int n = 0; n < NTOK; ++n) {
                    if (n >= valid) continue;
                    const int p = row0 + n;
                    if (DUAL) {
                        reinterpret_cast<__nv_bfloat16*>(y)[(size_t)p * ldy + m] =
                            __float2bfloat16_rn(moe_tc_act(acc[0][n], act) * acc[W_TILES - 1][n]);
                    } else if (row_dst == nullptr) {          // an expert without a gate: its hidden layer, act(up a_p)
                        reinterpret_cast<__nv_bfloat16*>(y)[(size_t)p * ldy + m] = __float2bfloat16_rn(moe_tc_act(acc[0][n], act));
                    } else {
                        const float v = row_w != nullptr ? acc[0][n] * row_w[p] : acc[0][n];
                        reinterpret_cast<float*>(y)[(size_t)row_dst[p] * ldy + m] = v;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) report_error(err, PRISM_ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS));
    }
}

template <int NTOK, bool DUAL>
int moe_launch(const void* x, long long ldx, long long x_rows, const void* W, const int* offs, const int* counts,
               const int* row_dst, const float* row_w, int token_tiles, int E, int N, int K, int act, void* y,
               long long ldy, int* err, cudaStream_t stream) {
    using C = MoeCfg<NTOK, DUAL>;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, (long long)E * (DUAL ? 2 : 1) * N, K, K, MOE_TILE_M);
    if (rc) return rc;
    rc = make_map(&mx, x, x_rows, K, ldx, NTOK);
    if (rc) return rc;
    auto kern = moe_swap_kernel<NTOK, DUAL>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    dim3 grid((N + MOE_TILE_M - 1) / MOE_TILE_M, token_tiles);
    return (int)launch_kernel(kern, grid, dim3(MOE_THREADS), C::SMEM, stream, mw, mx, offs, counts, row_dst, row_w, E, N, K, act,
                              y, ldy, err);
}

// One block per (token, choice): its row of x, times its weight (scale_in), rounded to bf16, at its padded place;
// and where the row's result goes.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x_in, long long ldx, const int* __restrict__ offs_in,
                                  const int* __restrict__ sel_e_in, const float* __restrict__ sel_w_in,
                                  const int* __restrict__ sel_rank_in, int T, int top, int W, int scale_in,
                                  __nv_bfloat16* __restrict__ xs, int* __restrict__ row_dst, float* __restrict__ row_w) {
    pdl_trigger();
    pdl_wait();
    const __nv_bfloat16* x = pdl_fresh(x_in);
    const int i = blockIdx.x;
    const int t = i / top, j = i - t * top;
    const int p = pdl_fresh(offs_in)[pdl_fresh(sel_e_in)[i]] + pdl_fresh(sel_rank_in)[i];
    const float w = pdl_fresh(sel_w_in)[i];
    if (threadIdx.x == 0) {
        row_dst[p] = j * T + t;
        row_w[p] = w;
    }
    const __nv_bfloat16* src = x + (size_t)t * ldx;
    __nv_bfloat16* dst = xs + (size_t)p * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = __bfloat162float(src[c]);
        dst[c] = scale_in ? __float2bfloat16_rn(v * w) : src[c];
    }
}

}  // namespace tc
}  // namespace prism

// 1 if the tensor-core path takes these sizes: bf16, rows of W and of the hidden layer 16 bytes aligned.
PRISM_EXPORT int prism_moe_tcgen05_supported(int W, int F) { return W >= 8 && F >= 8 && W % 8 == 0 && F % 8 == 0; }

// x [T, W] bf16 -> xs [padded rows, W] bf16 (row of (t, j) at offs[expert] + rank), row_dst and row_w at the same place.
// offs: the padded offsets that prism_moe_place made with pad = the token tile.
PRISM_EXPORT int prism_moe_gather(const void* x, long long ldx, const int* offs, const int* sel_e, const float* sel_w,
                                  const int* sel_rank, int T, int top, int W, int scale_in, void* xs, int* row_dst,
                                  float* row_w, cudaStream_t stream) {
    if (T <= 0) return 0;
    return (int)prism::launch_kernel(prism::tc::moe_gather_kernel, dim3(T * top), dim3(W >= 2048 ? 256 : 128), 0, stream,
                                     (const __nv_bfloat16*)x, ldx, offs, sel_e, sel_w, sel_rank, T, top, W, scale_in,
                                     (__nv_bfloat16*)xs, row_dst, row_w);
}

// a [x_rows, K] bf16 in padded order (x_rows = token_tiles * ntok); w [E, (2) N, K] bf16 contiguous.
// dual 1: out [x_rows, N] bf16 (row stride ldo), out[p] = act(gate a_p) * (up a_p).
// dual 0: out float32, out[row_dst[p]] = w a_p (times row_w[p] if row_w is given); row_dst null: out [x_rows, N] bf16,
// out[p] = act(w a_p).
PRISM_EXPORT int prism_moe_gemm_tcgen05(const void* a, long long lda, const void* w, const int* offs, const int* counts,
                                        const int* row_dst, const float* row_w, int ntok, int token_tiles, int E, int N,
                                        int K, int dual, int act, void* out, long long ldo, int* err, cudaStream_t stream) {
    using namespace prism::tc;
    if (token_tiles <= 0 || N <= 0) return 0;
    if (E < 1 || K < 8 || K % 8 || lda % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15) || token_tiles > 65535 ||
        (ntok != 16 && ntok != 32 && ntok != 64))
        return (int)cudaErrorInvalidValue;
    const long long x_rows = (long long)token_tiles * ntok;
#define ARGS a, lda, x_rows, w, offs, counts, row_dst, row_w, token_tiles, E, N, K, act, out, ldo, err, stream
    if (dual) return ntok == 16 ? moe_launch<16, true>(ARGS) : ntok == 32 ? moe_launch<32, true>(ARGS) : moe_launch<64, true>(ARGS);
    return ntok == 16 ? moe_launch<16, false>(ARGS) : ntok == 32 ? moe_launch<32, false>(ARGS) : moe_launch<64, false>(ARGS);
#undef ARGS
}
