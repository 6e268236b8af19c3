// Mixture of experts: every token goes through `top` of E small gated feed-forward layers, chosen by a router.
//   scores s = sigmoid(z) (or softmax(z)) of the float32 router logits z [T, E]; the `top` largest are taken (the
//   lower index wins a tie); the weight of a choice is its score, optionally divided by the sum of the chosen.
// The (token, choice) pairs are sorted by expert on the device, so that each expert's rows are one stretch:
//   prism_moe_route    top-k per token; counts[e] rows per expert, and each pair's rank among its expert's rows
//   prism_moe_route_place  both of the above in one CTA, for a step of few tokens
//   prism_moe_place    offs = prefix sums of counts (each rounded up to `pad`); per sorted row: its token, its weight,
//                      and where its result goes
//   prism_moe_gemm     grouped product over the sorted rows, expert by expert, no host knowledge of the counts:
//                      (dual)   hidden[p] = act(Wg[e] a_p) * (Wu[e] a_p),  a_p = x[token[p]] * (weight[p] or 1)
//                               (experts without a gate: hidden[p] = act(Wu[e] a_p))
//                      (single) y[dst[p]] = Wd[e] hidden[p] * (weight[p] or 1)
// The weight multiplies the expert's input (scale_in) or its output.  dst[p] = choice * T + token: the results of a
// token's choices land in `top` planes [top, T, W] that the next norm adds up in float32, in a fixed order.
// CUDA-core FFMA with float32 accumulation, k ascending inside one thread: a row's result does not depend on the
// batch around it.  bf16 operands are widened exactly, so the sums equal a tensor-core product's up to their order.
#include "common.cuh"

namespace prism {

__device__ __forceinline__ float moe_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float moe_act(float z, int act) {
    if (act == 0) return z / (1.f + expf(-z));                                                      // silu
    if (act == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));   // gelu_tanh
    const float r = fmaxf(z, 0.f);
    return act == 3 ? r * r : r;                                                                      // relu squared, relu
}

// One warp takes a token: scores into s [E] (shared), choice scores into c [E] (the score plus a correction per expert,
// where one is given), the `top` largest choice scores chosen (the lower index wins a tie), counts [E] (shared or global)
// raised by one per choice, whose old value is the choice's rank among its expert's rows.  With `groups` > 1 the experts
// form that many equal groups of neighbours, a group's score is its largest choice score, and only the experts of the
// best `keep` groups can be chosen (gs: 2 groups floats of scratch).  A choice's weight is its score without the
// correction, with renorm divided by the sum of the chosen (+ sum_eps), times wscale.
__device__ __forceinline__ void moe_route_token(const float* __restrict__ z, float* s, float* c, float* gs, int E, int top,
                                                int softmax, int renorm, int lane, int* counts, int* __restrict__ sel_e,
                                                float* __restrict__ sel_w, int* __restrict__ sel_rank,
                                                const void* __restrict__ corr, int corr_bf16, int groups, int keep,
                                                float wscale, float sum_eps) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = softmax ? expf(z[e] - mx) : moe_sigmoid(z[e]);
        s[e] = v;
        den += v;
    }
    den = warp_sum(den);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        const float v = softmax ? s[e] / den : s[e];
        s[e] = v;
        c[e] = corr != nullptr ? v + load_param(corr, corr_bf16, e) : v;
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        float* kept = gs + groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
            gs[g] = best;
            kept[g] = 0.f;
        }
        __syncwarp();
        for (int j = 0; j < keep; ++j) {
            float best = -INFINITY;
            int at = groups;
            for (int g = lane; g < groups; g += 32)
                if (kept[g] == 0.f && (gs[g] > best || at == groups)) { best = gs[g]; at = g; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa < groups && (at == groups || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (lane == 0 && at < groups) kept[at] = 1.f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (kept[e / per] == 0.f) c[e] = -INFINITY;
        __syncwarp();
    }
    float chosen = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32)
            if (c[e] > best) { best = c[e]; at = e; }           // ascending e: the lowest index of equal scores
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = 0;                                   // every score NaN: keep the indices legal
        const float w = s[at];
        chosen += w;
        if (lane == 0) {
            sel_e[j] = at;
            sel_w[j] = w;
            sel_rank[j] = atomicAdd(counts + at, 1);
            c[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0)
        for (int j = 0; j < top; ++j) sel_w[j] = (renorm ? sel_w[j] / (chosen + sum_eps) : sel_w[j]) * wscale;
}

// One warp per token.  logits [T, E] float32 (row stride ls).  sel_e, sel_w, sel_rank [T, top].
__global__ void moe_route_kernel(const float* __restrict__ logits_in, long long ls, int T, int E, int top, int softmax,
                                 int renorm, int* __restrict__ counts, int* __restrict__ sel_e, float* __restrict__ sel_w,
                                 int* __restrict__ sel_rank, const void* __restrict__ corr, int corr_bf16, int groups, int keep,
                                 float wscale, float sum_eps) {
    pdl_trigger();
    pdl_wait();
    const float* logits = pdl_fresh(logits_in);
    extern __shared__ float sc[];                       // [warps][2 E + 2 groups]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* mine = sc + (size_t)warp * (2 * E + 2 * groups);
    moe_route_token(logits + (size_t)t * ls, mine, mine + E, mine + 2 * E, E, top, softmax, renorm, lane, counts,
                    sel_e + (size_t)t * top, sel_w + (size_t)t * top, sel_rank + (size_t)t * top, corr, corr_bf16, groups, keep,
                    wscale, sum_eps);
}

// A step of few tokens (decode) in one CTA and one launch: the counters start at zero in shared memory, a warp routes
// every eighth token, then the offsets (stretches padded to `pad`) and, unless row_tok is null, the sorted rows.
__global__ void moe_route_place_kernel(const float* __restrict__ logits_in, long long ls, int T, int E, int top, int softmax,
                                       int renorm, int pad, int* __restrict__ counts_out, int* __restrict__ offs,
                                       int* __restrict__ sel_e, float* __restrict__ sel_w, int* __restrict__ sel_rank,
                                       int* __restrict__ row_tok, float* __restrict__ row_w, int* __restrict__ row_dst,
                                       const void* __restrict__ corr, int corr_bf16, int groups, int keep, float wscale,
                                       float sum_eps) {
    pdl_trigger();
    extern __shared__ float sc[];                       // [warps][2 E + 2 groups] floats, then counts [E] and offsets [E + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int per_warp = 2 * E + 2 * groups;
    int* cnt = reinterpret_cast<int*>(sc + (size_t)warps * per_warp);
    int* so = cnt + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    pdl_wait();
    const float* logits = pdl_fresh(logits_in);
    __syncthreads();
    float* mine = sc + (size_t)warp * per_warp;
    for (int t = warp; t < T; t += warps)
        moe_route_token(logits + (size_t)t * ls, mine, mine + E, mine + 2 * E, E, top, softmax, renorm, lane, cnt,
                        sel_e + (size_t)t * top, sel_w + (size_t)t * top, sel_rank + (size_t)t * top, corr, corr_bf16, groups,
                        keep, wscale, sum_eps);
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            so[e] = acc;
            acc += (cnt[e] + pad - 1) / pad * pad;
        }
        so[E] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) {
        offs[e] = so[e];
        if (e < E) counts_out[e] = cnt[e];
    }
    if (row_tok == nullptr) return;
    for (int i = threadIdx.x; i < T * top; i += blockDim.x) {
        const int t = i / top, j = i - t * top;
        const int p = so[sel_e[i]] + sel_rank[i];
        row_tok[p] = t;
        row_w[p] = sel_w[i];
        row_dst[p] = j * T + t;
    }
}

// offs [E + 1]: every expert's stretch starts at a multiple of pad; row_tok, row_w, row_dst in sorted order (at the
// padded places), or none of the three when row_tok is null.
__global__ void moe_place_kernel(const int* __restrict__ counts_in, const int* __restrict__ sel_e_in,
                                 const float* __restrict__ sel_w_in, const int* __restrict__ sel_rank_in, int T, int E, int top,
                                 int pad, int* __restrict__ offs, int* __restrict__ row_tok, float* __restrict__ row_w,
                                 int* __restrict__ row_dst) {
    pdl_trigger();
    pdl_wait();
    const int* counts = pdl_fresh(counts_in);
    const int* sel_e = pdl_fresh(sel_e_in);
    const float* sel_w = pdl_fresh(sel_w_in);
    const int* sel_rank = pdl_fresh(sel_rank_in);
    extern __shared__ int so[];                          // [E + 1]
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            so[e] = acc;
            acc += (counts[e] + pad - 1) / pad * pad;
        }
        so[E] = acc;
    }
    __syncthreads();
    if (blockIdx.x == 0)
        for (int e = threadIdx.x; e <= E; e += blockDim.x) offs[e] = so[e];
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * top || row_tok == nullptr) return;
    const int t = i / top, j = i - t * top;
    const int p = so[sel_e[i]] + sel_rank[i];
    row_tok[p] = t;
    row_w[p] = sel_w[i];
    row_dst[p] = j * T + t;
}

// Grouped product over the sorted rows.  A [*, K] of AT (row stride lda): DUAL reads row row_tok[p] (times row_w[p] with
// scale_in, rounded to AT), single reads row p.  W [E, N (x2 for DUAL: the gate's rows, then the up's), K] of AT.
// DUAL: out [T top, N] of AT at row p.  single: out [top T, N] float32 at row row_dst[p] (times row_w[p] without
// scale_in).  grid (N tiles, row tiles): row tile i belongs to the expert whose tiles of BM rows cover it.
template <typename AT, bool DUAL, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
moe_gemm_kernel(const AT* __restrict__ A_in, long long lda, const AT* __restrict__ W, const int* __restrict__ offs_in,
                const int* __restrict__ row_tok_in, const float* __restrict__ row_w_in, const int* __restrict__ row_dst_in, int E,
                int N, int K, int scale_in, int act, void* __restrict__ out, long long ldo, int gated) {
    pdl_trigger();
    pdl_wait();
    const AT* A = pdl_fresh(A_in);
    const int* offs = pdl_fresh(offs_in);
    const int* row_tok = pdl_fresh(row_tok_in);
    const float* row_w = pdl_fresh(row_w_in);
    const int* row_dst = pdl_fresh(row_dst_in);
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[DUAL ? BK : 1][BN + 4];
    __shared__ int rows_src[BM];
    __shared__ float rows_w[BM];
    __shared__ int tile_info[3];
    const int tid = threadIdx.x;
    if (tid == 0) {
        int idx = blockIdx.y, e = 0, found = -1, m0 = 0;
        for (; e < E; ++e) {
            const int c = offs[e + 1] - offs[e];
            const int tiles = (c + BM - 1) / BM;
            if (idx < tiles) {
                found = e;
                m0 = offs[e] + idx * BM;
                break;
            }
            idx -= tiles;
        }
        tile_info[0] = found;
        tile_info[1] = m0;
        tile_info[2] = found >= 0 ? offs[found + 1] : 0;
    }
    __syncthreads();
    const int e = tile_info[0], m0 = tile_info[1], mend = tile_info[2];
    if (e < 0) return;
    for (int r = tid; r < BM; r += THREADS) {
        const int p = m0 + r;
        rows_src[r] = p < mend ? (DUAL ? row_tok[p] : p) : -1;
        rows_w[r] = p < mend ? row_w[p] : 0.f;
    }
    __syncthreads();
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int n0 = blockIdx.x * BN;
    const AT* We = W + (size_t)e * ((DUAL && gated) ? 2 : 1) * N * K;
    const AT* Wu = We + (size_t)N * K;
    float acc[TM][TN], acu[DUAL ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (DUAL) acu[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = tid; idx < BM * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            const int src = rows_src[r];
            float v = 0.f;
            if (src >= 0 && k0 + c < K) {
                v = to_float(A[(size_t)src * lda + k0 + c]);
                if (DUAL && scale_in) v = to_float(from_float<AT>(v * rows_w[r]));
            }
            As[c][r] = v;
        }
        for (int idx = tid; idx < BN * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            const bool ok = n0 + r < N && k0 + c < K;
            Ws[c][r] = ok ? to_float(We[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
            if (DUAL && gated) Us[c][r] = ok ? to_float(Wu[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN], u[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                b[j] = Ws[kk][tx * TN + j];
                if (DUAL) u[j] = Us[kk][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (DUAL) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        const int p = m0 + r;
        if (p >= mend) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            if (DUAL) {
                reinterpret_cast<AT*>(out)[(size_t)p * ldo + n] =
                    from_float<AT>(gated ? moe_act(acc[i][j], act) * acu[i][j] : moe_act(acc[i][j], act));
            } else {
                reinterpret_cast<float*>(out)[(size_t)row_dst[p] * ldo + n] = scale_in ? acc[i][j] : acc[i][j] * rows_w[r];
            }
        }
    }
}

}  // namespace prism

// logits [T, E] float32; counts [E] int32, zero before the call; sel_e, sel_rank int32 and sel_w float32 [T, top].
PRISM_EXPORT int prism_moe_route(const float* logits, long long logits_stride, int T, int E, int top, int softmax, int renorm,
                                 int* counts, int* sel_e, float* sel_w, int* sel_rank, const void* corr, int corr_dtype,
                                 int groups, int keep, float wscale, float sum_eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E < 1 || top < 1 || top > E) return (int)cudaErrorInvalidValue;
    if (groups < 1 || E % groups || keep < 1 || keep > groups || keep * (E / groups) < top) return (int)cudaErrorInvalidValue;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + 2 * groups) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kern = prism::moe_route_kernel;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)prism::launch_kernel(kern, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, stream, logits, logits_stride,
                                     T, E, top, softmax, renorm, counts, sel_e, sel_w, sel_rank, corr,
                                     corr_dtype == PRISM_DTYPE_BF16, groups, keep, wscale, sum_eps);
}

// prism_moe_route and prism_moe_place (and the counters' reset) in one launch of one CTA, for steps of few tokens.
PRISM_EXPORT int prism_moe_route_place(const float* logits, long long logits_stride, int T, int E, int top, int softmax,
                                       int renorm, int pad, int* counts, int* offs, int* sel_e, float* sel_w, int* sel_rank,
                                       int* row_tok, float* row_w, int* row_dst, const void* corr, int corr_dtype, int groups,
                                       int keep, float wscale, float sum_eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E < 1 || top < 1 || top > E || pad < 1) return (int)cudaErrorInvalidValue;
    if (groups < 1 || E % groups || keep < 1 || keep > groups || keep * (E / groups) < top) return (int)cudaErrorInvalidValue;
    const int warps = 8;
    const size_t smem = (size_t)warps * (2 * E + 2 * groups) * sizeof(float) + (size_t)(2 * E + 1) * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return (int)prism::launch_kernel(prism::moe_route_place_kernel, dim3(1), dim3(32 * warps), smem, stream, logits,
                                     logits_stride, T, E, top, softmax, renorm, pad, counts, offs, sel_e, sel_w, sel_rank,
                                     row_tok, row_w, row_dst, corr, corr_dtype == PRISM_DTYPE_BF16, groups, keep, wscale, sum_eps);
}

PRISM_EXPORT int prism_moe_place(const int* counts, const int* sel_e, const float* sel_w, const int* sel_rank, int T, int E,
                                 int top, int pad, int* offs, int* row_tok, float* row_w, int* row_dst, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (pad < 1) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(E + 1) * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return (int)prism::launch_kernel(prism::moe_place_kernel, dim3((T * top + 255) / 256), dim3(256), smem, stream, counts, sel_e,
                                     sel_w, sel_rank, T, E, top, pad, offs, row_tok, row_w, row_dst);
}

// rows = T top sorted rows.  dual 1: a [T, K], w [E, 2 N, K], out [rows, N] of dtype; dual 0: a [rows, K], w [E, N, K],
// out [rows, N] float32 (written at row_dst).  act: 0 silu, 1 gelu_tanh, 2 relu, 3 relu squared.  gated 0 (with dual 1):
// w [E, N, K] and out[p] = act(w a_p), an expert without a gate.
PRISM_EXPORT int prism_moe_gemm(const void* a, long long lda, const void* w, int dtype, const int* offs, const int* row_tok,
                                const float* row_w, const int* row_dst, int rows, int E, int N, int K, int dual, int scale_in,
                                int act, void* out, long long ldo, int gated, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return 0;
    if (E < 1 || K < 1) return (int)cudaErrorInvalidValue;
#define PRISM_MG(AT, D, BM, BN, BK, TM, TN)                                                                              \
    do {                                                                                                                 \
        long long tiles = (rows + BM - 1) / BM + E;                                                                      \
        if (tiles > rows) tiles = rows;                                                                                  \
        if (tiles > 65535) return (int)cudaErrorInvalidValue;                                                            \
        dim3 grid((N + BN - 1) / BN, (unsigned)tiles);                                                                   \
        return (int)prism::launch_kernel(prism::moe_gemm_kernel<AT, D, BM, BN, BK, TM, TN>, grid,                         \
                                         dim3((BM / TM) * (BN / TN)), 0, stream, (const AT*)a, lda, (const AT*)w, offs,   \
                                         row_tok, row_w, row_dst, E, N, K, scale_in, act, out, ldo, gated);              \
    } while (0)
    const bool few = rows <= 16 * E / 2 || rows <= 64;       // most experts see under a tile's worth of rows
    if (dtype == PRISM_DTYPE_BF16) {
        if (dual) {
            if (few) PRISM_MG(__nv_bfloat16, true, 16, 32, 32, 1, 2);
            PRISM_MG(__nv_bfloat16, true, 64, 32, 16, 4, 2);
        }
        if (few) PRISM_MG(__nv_bfloat16, false, 16, 64, 32, 1, 4);
        PRISM_MG(__nv_bfloat16, false, 64, 64, 16, 4, 4);
    }
    if (dual) {
        if (few) PRISM_MG(float, true, 16, 32, 32, 1, 2);
        PRISM_MG(float, true, 64, 32, 16, 4, 2);
    }
    if (few) PRISM_MG(float, false, 16, 64, 32, 1, 4);
    PRISM_MG(float, false, 64, 64, 16, 4, 4);
#undef PRISM_MG
}
