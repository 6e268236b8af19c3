// Real-gated linear recurrent unit: a recurrence with one float32 number of state per channel,
//     S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t,      a_t = exp(-c r_t softplus(lam)),
// whose gates r and i are sigmoids of block-diagonal products of u (the channels are split into equal blocks,
// each with a square matrix for r and one for i).  Three kernels:
//   * prism_causal_conv   u = conv(x) + bias: the short causal convolution over time per channel (its last taps - 1
//     inputs per request are state too; a step of single tokens moves that tail up itself);
//   * prism_block_gates   both block-diagonal products with the recurrence's coefficients as epilogue: from u it
//     writes a and sqrt(1 - a^2) i u, float32 throughout (CUDA cores, k ascending inside one thread, so a row's
//     result does not depend on the batch);
//   * prism_rglru_scan    the recurrence itself from and into the request's state slot, token after token, times
//     the other branch's activation, rounded once to the compute dtype.
#include "common.cuh"

namespace prism {

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rg_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rg_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out[t][c] = bias[c] + sum_j taps[c][K-1-j] x[t-j][c] (+ x[t][c] with add_input: a convolution beside a skip path);
// x [T, *] float32 with row stride xs; tail [slots, K-1, C]; out float32 or the compute dtype (rounded once).
// taps_t (or null): the same taps as float32 [K, C], which the vector path reads 128 bits at a time.
// One CTA per token: it looks up the token's segment, place and slot once, and its threads walk the channels VEC at a
// time (one 128-bit load a row with VEC 4), the loads of one pass independent of the next pass's.
template <typename TO, int VEC>
__global__ void causal_conv_kernel(const float* __restrict__ x_in, long long xs, const void* __restrict__ taps, int taps_bf16,
                                   const void* __restrict__ bias, int bias_bf16, int K, int C, float* tail,
                                   const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                                   const int* __restrict__ slots, TO* __restrict__ out, long long os, int move_tail,
                                   int add_input, const float* __restrict__ taps_t) {
    pdl_trigger();
    const int t = blockIdx.x, seg = tok_seg[t];        // the step's descriptor is complete before the step's first kernel
    const int i = t - seg_start[seg];
    float* tl = tail + (size_t)slots[seg] * (K - 1) * C;
    pdl_wait();
    const float* x = pdl_fresh(x_in);
#pragma unroll 2
    for (int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c0 < C; c0 += gridDim.y * blockDim.x * VEC) {
        float acc[VEC], cur[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = bias != nullptr ? load_param(bias, bias_bf16, c0 + v) : 0.f;
        for (int j = K - 1; j >= 0; --j) {             // lag j: the input j tokens back; oldest first
            const int src = i - j;
            const float* row = src >= 0 ? x + (size_t)(t - j) * xs + c0 : tl + (size_t)(K - 1 + src) * C + c0;
            float val[VEC];
            if (VEC == 4) {
                const float4 q = *reinterpret_cast<const float4*>(row);
                val[0] = q.x; val[1 % VEC] = q.y; val[2 % VEC] = q.z; val[3 % VEC] = q.w;
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) val[v] = row[v];
            }
            float w[VEC];
            if (VEC == 4 && taps_t != nullptr) {       // the taps turned to [K, C] float32: one 128-bit load a lag
                const float4 q = *reinterpret_cast<const float4*>(taps_t + (size_t)(K - 1 - j) * C + c0);
                w[0] = q.x; w[1 % VEC] = q.y; w[2 % VEC] = q.z; w[3 % VEC] = q.w;
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) w[v] = load_param(taps, taps_bf16, (size_t)(c0 + v) * K + (K - 1 - j));
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                acc[v] += w[v] * val[v];
                if (j == 0) cur[v] = val[v];
            }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) out[(size_t)t * os + c0 + v] = from_float<TO>(add_input ? acc[v] + cur[v] : acc[v]);
        if (move_tail && K > 1) {          // one token per request: this thread is the only reader of its channels' tail
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                for (int r = 0; r + 2 < K; ++r) tl[(size_t)r * C + c0 + v] = tl[(size_t)(r + 1) * C + c0 + v];
                tl[(size_t)(K - 2) * C + c0 + v] = cur[v];
            }
        }
    }
}

// The same convolution for portions of prompts where the sizes allow 128-bit accesses, the taps are given as float32
// [K, C] and K <= CONVT_TAPS: a CTA takes CONVT_TOK consecutive tokens of the step.  Their segments, places and slots are
// looked up side by side first; a thread then loads its four channels of all CONVT_TOK rows (independent loads) and of the
// taps once, and serves every lag from those registers where the lag stays inside the tile and the token's segment, from
// the rows before the tile or from the request's tail otherwise - in the order of the one-token kernel, so both give the
// same sums.  A row is read from L2 about (CONVT_TOK + K - 1) / CONVT_TOK times instead of K times.
constexpr int CONVT_TOK = 8;
constexpr int CONVT_TAPS = 8;
template <typename TO>
__global__ void causal_conv_tile_kernel(const float* __restrict__ x_in, long long xs, const float* __restrict__ taps_t,
                                        const void* __restrict__ bias, int bias_bf16, int K, int C, const float* tail,
                                        const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                                        const int* __restrict__ slots, TO* __restrict__ out, long long os, int add_input, int T) {
    pdl_trigger();
    __shared__ int s_place[CONVT_TOK], s_slot[CONVT_TOK];
    const int t0 = blockIdx.x * CONVT_TOK;
    if (threadIdx.x < CONVT_TOK) {                       // the step's descriptor is complete before the step's first kernel
        const int t = t0 + threadIdx.x;
        const int seg = t < T ? tok_seg[t] : 0;
        s_place[threadIdx.x] = t < T ? t - seg_start[seg] : 0;
        s_slot[threadIdx.x] = slots[seg];
    }
    __syncthreads();
    pdl_wait();
    const float* x = pdl_fresh(x_in);
    for (int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c0 < C; c0 += gridDim.y * blockDim.x * 4) {
        float4 w[CONVT_TAPS], xr[CONVT_TOK];
#pragma unroll
        for (int j = 0; j < CONVT_TAPS; ++j)            // w[j]: the tap of lag j
            w[j] = j < K ? *reinterpret_cast<const float4*>(taps_t + (size_t)(K - 1 - j) * C + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int tt = 0; tt < CONVT_TOK; ++tt)
            xr[tt] = t0 + tt < T ? *reinterpret_cast<const float4*>(x + (size_t)(t0 + tt) * xs + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias != nullptr)
            b4 = make_float4(load_param(bias, bias_bf16, c0), load_param(bias, bias_bf16, c0 + 1), load_param(bias, bias_bf16, c0 + 2),
                             load_param(bias, bias_bf16, c0 + 3));
#pragma unroll
        for (int tt = 0; tt < CONVT_TOK; ++tt) {
            const int t = t0 + tt;
            if (t >= T) break;
            const int i = s_place[tt];
            const float* tl = tail + (size_t)s_slot[tt] * (K - 1) * C + c0;
            float4 acc = b4;
#pragma unroll
            for (int j = CONVT_TAPS - 1; j >= 0; --j) {   // oldest first
                if (j >= K) continue;
                float4 v;
                if (j <= i) {
                    if (tt - j >= 0) v = xr[tt - j >= 0 ? tt - j : 0];
                    else v = *reinterpret_cast<const float4*>(x + (size_t)(t - j) * xs + c0);
                } else {
                    v = *reinterpret_cast<const float4*>(tl + (size_t)(K - 1 + i - j) * C);
                }
                acc.x += w[j].x * v.x; acc.y += w[j].y * v.y; acc.z += w[j].z * v.z; acc.w += w[j].w * v.w;
            }
            if (add_input) { acc.x += xr[tt].x; acc.y += xr[tt].y; acc.z += xr[tt].z; acc.w += xr[tt].w; }
            TO* o = out + (size_t)t * os + c0;
            o[0] = from_float<TO>(acc.x); o[1] = from_float<TO>(acc.y); o[2] = from_float<TO>(acc.z); o[3] = from_float<TO>(acc.w);
        }
    }
}

// Block b of channels [b bs, (b + 1) bs): r = sigmoid(Wr[b] u_b + br[b]), i = sigmoid(Wi[b] u_b + bi[b]);
// a = exp(-c r softplus(lam)), g = sqrt(1 - a^2) i u.  Wr, Wi [blocks, bs, bs] ([out, in]); grid (bs tiles, token tiles,
// blocks).  1 - a^2 is formed as -expm1(2 log a), which keeps its leading digits where a is close to 1.
template <typename WT, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
block_gates_kernel(const float* __restrict__ u_in, long long us, const WT* __restrict__ Wr, const WT* __restrict__ Wi,
                   const void* __restrict__ br, const void* __restrict__ bi, int b_bf16, const void* __restrict__ lam,
                   int lam_bf16, float cdecay, int T, int bs, float* __restrict__ a_out, float* __restrict__ g_out,
                   long long os) {
    pdl_trigger();
    pdl_wait();
    const float* u = pdl_fresh(u_in);
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Rs[BK][BN + 4];
    __shared__ float Is[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int blk = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const size_t wbase = (size_t)blk * bs * bs;
    const float* ub = u + (size_t)blk * bs;
    float ar[TM][TN], ai[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) ar[i][j] = ai[i][j] = 0.f;
    for (int k0 = 0; k0 < bs; k0 += BK) {
        for (int idx = tid; idx < BM * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            As[c][r] = (m0 + r < T && k0 + c < bs) ? ub[(size_t)(m0 + r) * us + k0 + c] : 0.f;
        }
        for (int idx = tid; idx < BN * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            const bool ok = n0 + r < bs && k0 + c < bs;
            const size_t at = wbase + (size_t)(n0 + r) * bs + k0 + c;
            Rs[c][r] = ok ? to_float(Wr[at]) : 0.f;
            Is[c][r] = ok ? to_float(Wi[at]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], r[TN], ii[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                r[j] = Rs[kk][tx * TN + j];
                ii[j] = Is[kk][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    ar[i][j] = fmaf(a[i], r[j], ar[i][j]);
                    ai[i][j] = fmaf(a[i], ii[j], ai[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= T) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= bs) continue;
            const size_t ch = (size_t)blk * bs + n;
            const float r = rg_sigmoid(ar[i][j] + load_param(br, b_bf16, ch));
            const float gi = rg_sigmoid(ai[i][j] + load_param(bi, b_bf16, ch));
            const float loga = -cdecay * r * rg_softplus(load_param(lam, lam_bf16, ch));
            a_out[(size_t)m * os + ch] = expf(loga);
            g_out[(size_t)m * os + ch] = sqrtf(-expm1f(2.f * loga)) * gi * ub[(size_t)m * us + n];
        }
    }
}

// S <- a S + g per channel, token after token of each request of the step; out = S * gelu_tanh(y) (act 1) or S * y.
// grid (channel blocks, segments); a thread owns a channel.  The loads of the next tokens do not depend on S, so
// they are issued four tokens ahead of the chain of multiply-adds.
template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ a_in, const float* __restrict__ g_in, long long as,
                                  const float* __restrict__ y_in, long long ys, float* __restrict__ state,
                                  const int* __restrict__ seg_start, const int* __restrict__ slots, int C, int act,
                                  T* __restrict__ out, long long os) {
    pdl_trigger();
    pdl_wait();
    const float* a = pdl_fresh(a_in);
    const float* g = pdl_fresh(g_in);
    const float* y = pdl_fresh(y_in);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seg = blockIdx.y, s0 = seg_start[seg], s1 = seg_start[seg + 1];
    float* st = state + (size_t)slots[seg] * C + c;
    float S = *st;
    int t = s0;
    for (; t + 4 <= s1; t += 4) {
        float av[4], gv[4], yv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            av[j] = a[(size_t)(t + j) * as + c];
            gv[j] = g[(size_t)(t + j) * as + c];
            yv[j] = y[(size_t)(t + j) * ys + c];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            S = fmaf(av[j], S, gv[j]);
            out[(size_t)(t + j) * os + c] = from_float<T>(S * (act ? rg_gelu_tanh(yv[j]) : yv[j]));
        }
    }
    for (; t < s1; ++t) {
        S = fmaf(a[(size_t)t * as + c], S, g[(size_t)t * as + c]);
        const float yv = y[(size_t)t * ys + c];
        out[(size_t)t * os + c] = from_float<T>(S * (act ? rg_gelu_tanh(yv) : yv));
    }
    *st = S;
}

// The same recurrence for long stretches, in two launches.  A request's tokens are cut into chunks of L; chunk k of
// request i keeps its results in row  seg_start[i] / L + i + k  of ws [rows, 2, C] (no two requests share a row).
//   pass 1, per chunk and channel:  A = product of a,  B = the chunk's last S when it starts from 0;  chunk 0 also
//                                   saves the state the request came with (ws0 [S, C]).
//   pass 2, per chunk and channel:  S = the saved state, carried over the chunks before this one (S <- A S + B),
//                                   then the chunk itself, token after token; the last chunk leaves the state.
// grid (channel blocks, chunks of the longest request, requests).
template <int L>
__global__ void rglru_chunk_kernel(const float* __restrict__ a_in, const float* __restrict__ g_in, long long as,
                                   const float* __restrict__ state_in, const int* __restrict__ seg_start,
                                   const int* __restrict__ slots, int C, float* __restrict__ ws, float* __restrict__ ws0) {
    pdl_trigger();
    pdl_wait();
    const float* a = pdl_fresh(a_in);
    const float* g = pdl_fresh(g_in);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seg = blockIdx.z, s0 = seg_start[seg], s1 = seg_start[seg + 1];
    const int t0 = s0 + blockIdx.y * L;
    if (t0 >= s1) return;
    const int t1 = min(s1, t0 + L);
    if (blockIdx.y == 0) ws0[(size_t)seg * C + c] = pdl_fresh(state_in)[(size_t)slots[seg] * C + c];
    float A = 1.f, B = 0.f;
    int t = t0;
    for (; t + 4 <= t1; t += 4) {
        float av[4], gv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            av[j] = a[(size_t)(t + j) * as + c];
            gv[j] = g[(size_t)(t + j) * as + c];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            A *= av[j];
            B = fmaf(av[j], B, gv[j]);
        }
    }
    for (; t < t1; ++t) {
        const float av = a[(size_t)t * as + c];
        A *= av;
        B = fmaf(av, B, g[(size_t)t * as + c]);
    }
    float* w = ws + ((size_t)(s0 / L + seg + blockIdx.y) * 2) * C + c;
    w[0] = A;
    w[C] = B;
}

template <typename T, int L>
__global__ void rglru_apply_kernel(const float* __restrict__ a_in, const float* __restrict__ g_in, long long as,
                                   const float* __restrict__ y_in, long long ys, float* __restrict__ state,
                                   const int* __restrict__ seg_start, const int* __restrict__ slots, int C, int act,
                                   const float* __restrict__ ws_in, const float* __restrict__ ws0_in, T* __restrict__ out,
                                   long long os) {
    pdl_trigger();
    pdl_wait();
    const float* a = pdl_fresh(a_in);
    const float* g = pdl_fresh(g_in);
    const float* y = pdl_fresh(y_in);
    const float* ws = pdl_fresh(ws_in);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seg = blockIdx.z, s0 = seg_start[seg], s1 = seg_start[seg + 1];
    const int t0 = s0 + blockIdx.y * L;
    if (t0 >= s1) return;
    const int t1 = min(s1, t0 + L);
    float S = pdl_fresh(ws0_in)[(size_t)seg * C + c];
    const float* w = ws + ((size_t)(s0 / L + seg) * 2) * C + c;
    for (int k = 0; k < (int)blockIdx.y; ++k, w += 2 * (size_t)C) S = fmaf(w[0], S, w[C]);
    int t = t0;
    for (; t + 4 <= t1; t += 4) {
        float av[4], gv[4], yv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            av[j] = a[(size_t)(t + j) * as + c];
            gv[j] = g[(size_t)(t + j) * as + c];
            yv[j] = y[(size_t)(t + j) * ys + c];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            S = fmaf(av[j], S, gv[j]);
            out[(size_t)(t + j) * os + c] = from_float<T>(S * (act ? rg_gelu_tanh(yv[j]) : yv[j]));
        }
    }
    for (; t < t1; ++t) {
        S = fmaf(a[(size_t)t * as + c], S, g[(size_t)t * as + c]);
        const float yv = y[(size_t)t * ys + c];
        out[(size_t)t * os + c] = from_float<T>(S * (act ? rg_gelu_tanh(yv) : yv));
    }
    if (t1 == s1) state[(size_t)slots[seg] * C + c] = S;
}

}  // namespace prism

PRISM_EXPORT int prism_causal_conv(const float* x, long long x_stride, const void* taps, int taps_dtype, const void* bias,
                                   int bias_dtype, int K, int C, float* tail, const int* tok_seg, const int* seg_start,
                                   const int* slots, int T, void* out, int out_dtype, long long out_stride, int move_tail,
                                   int add_input, const float* taps_t, cudaStream_t stream) {
    using namespace prism;
    if (T <= 0 || C <= 0) return 0;
    if (taps_t != nullptr && (uintptr_t)taps_t % 16 != 0) taps_t = nullptr;
    if (K < 1) return (int)cudaErrorInvalidValue;
    // 128-bit loads where every row piece starts on 16 bytes
    const bool vec = C % 4 == 0 && x_stride % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)tail % 16 == 0;
    const int per = vec ? 4 : 1;
    const int groups = (C + per - 1) / per;
    const int threads = groups >= 256 ? 256 : (groups >= 128 ? 128 : (groups >= 64 ? 64 : 32));
    // a step of few tokens: several CTAs share a token's channels, so that the GPU is not left to a handful of CTAs
    int gy = 1;
    while (T * gy < 128 && gy * threads * 2 <= groups) gy *= 2;
    const dim3 grid(T, gy);
    const int tb = taps_dtype == PRISM_DTYPE_BF16, bb = bias_dtype == PRISM_DTYPE_BF16;
    // portions of prompts: tiles of tokens whose rows and taps stay in registers
    if (vec && !move_tail && taps_t != nullptr && K <= CONVT_TAPS && T >= 2 * CONVT_TOK && out_stride % 4 == 0) {
        int ty = 1;
        const int tiles = (T + CONVT_TOK - 1) / CONVT_TOK;
        while (tiles * ty < 296 && ty * 128 * 2 <= groups) ty *= 2;
        const dim3 tgrid(tiles, ty);
        const int tthreads = groups / ty >= 128 ? 128 : (groups / ty >= 64 ? 64 : 32);
        if (out_dtype == PRISM_DTYPE_BF16)
            return (int)launch_kernel(causal_conv_tile_kernel<__nv_bfloat16>, tgrid, dim3(tthreads), 0, stream, x, x_stride, taps_t, bias,
                                      bb, K, C, (const float*)tail, tok_seg, seg_start, slots, (__nv_bfloat16*)out, out_stride,
                                      add_input, T);
        return (int)launch_kernel(causal_conv_tile_kernel<float>, tgrid, dim3(tthreads), 0, stream, x, x_stride, taps_t, bias, bb, K, C,
                                  (const float*)tail, tok_seg, seg_start, slots, (float*)out, out_stride, add_input, T);
    }
#define PRISM_CONV(TO, V)                                                                                               \
    return (int)launch_kernel(causal_conv_kernel<TO, V>, grid, dim3(threads), 0, stream, x, x_stride, taps, tb, bias, bb, K, C, \
                              tail, tok_seg, seg_start, slots, (TO*)out, out_stride, move_tail, add_input, taps_t)
    if (out_dtype == PRISM_DTYPE_BF16) {
        if (vec) PRISM_CONV(__nv_bfloat16, 4);
        PRISM_CONV(__nv_bfloat16, 1);
    }
    if (vec) PRISM_CONV(float, 4);
    PRISM_CONV(float, 1);
#undef PRISM_CONV
}

// u [T, blocks * bs] float32 (row stride u_stride); wr, wi [blocks, bs, bs] of w_dtype; br, bi [blocks * bs] of b_dtype;
// lam [blocks * bs]; a_out, g_out [T, blocks * bs] float32 with row stride out_stride.
PRISM_EXPORT int prism_block_gates(const float* u, long long u_stride, const void* wr, const void* wi, int w_dtype,
                                   const void* br, const void* bi, int b_dtype, const void* lam, int lam_dtype, float cdecay,
                                   int T, int blocks, int bs, float* a_out, float* g_out, long long out_stride,
                                   cudaStream_t stream) {
    if (T <= 0) return 0;
    if (blocks < 1 || bs < 1 || blocks > 65535) return (int)cudaErrorInvalidValue;
    const int bb = b_dtype == PRISM_DTYPE_BF16, lb = lam_dtype == PRISM_DTYPE_BF16;
#define PRISM_BG(WT, BM, BK, TM)                                                                                        \
    do {                                                                                                                \
        dim3 grid((bs + 31) / 32, (T + BM - 1) / BM, blocks);                                                           \
        if (grid.y > 65535) return (int)cudaErrorInvalidValue;                                                          \
        return (int)prism::launch_kernel(prism::block_gates_kernel<WT, BM, 32, BK, TM, 2>, grid, dim3((BM / TM) * 16), 0, \
                                         stream, u, u_stride, (const WT*)wr, (const WT*)wi, br, bi, bb, lam, lb, cdecay, T, \
                                         bs, a_out, g_out, out_stride);                                                 \
    } while (0)
    if (w_dtype == PRISM_DTYPE_BF16) {
        if (T <= 16) PRISM_BG(__nv_bfloat16, 16, 32, 1);
        PRISM_BG(__nv_bfloat16, 64, 16, 4);
    }
    if (T <= 16) PRISM_BG(float, 16, 32, 1);
    PRISM_BG(float, 64, 16, 4);
#undef PRISM_BG
}

// a, g [T, C] float32 (one row stride), y [T, C] float32 (row stride y_stride), state [slots, C] float32,
// out [T, C] of out_dtype; act 1: gelu_tanh(y), 0: y as it is.
PRISM_EXPORT int prism_rglru_scan(const float* a, const float* g, long long ag_stride, const float* y, long long y_stride,
                                  float* state, const int* seg_start, const int* slots, int S, int C, int act, void* out,
                                  int out_dtype, long long out_stride, cudaStream_t stream) {
    if (S <= 0 || C <= 0) return 0;
    if (S > 65535) return (int)cudaErrorInvalidValue;
    const int threads = (long long)S * C >= 148 * 256 ? 128 : 32;       // few requests: more, smaller CTAs
    dim3 grid((C + threads - 1) / threads, S);
    if (out_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::rglru_scan_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, a, g, ag_stride,
                                         y, y_stride, state, seg_start, slots, C, act, (__nv_bfloat16*)out, out_stride);
    return (int)prism::launch_kernel(prism::rglru_scan_kernel<float>, grid, dim3(threads), 0, stream, a, g, ag_stride, y,
                                     y_stride, state, seg_start, slots, C, act, (float*)out, out_stride);
}

#define PRISM_RGLRU_CHUNK 64

// The chunked form for long stretches: longest = the longest request's tokens in this step (an upper bound will do);
// ws: float32 [T / 64 + S + 1, 2, C], ws0: float32 [S, C].
PRISM_EXPORT int prism_rglru_scan_chunked(const float* a, const float* g, long long ag_stride, const float* y,
                                          long long y_stride, float* state, const int* seg_start, const int* slots, int S,
                                          int C, int longest, int act, float* ws, float* ws0, void* out, int out_dtype,
                                          long long out_stride, cudaStream_t stream) {
    if (S <= 0 || C <= 0 || longest <= 0) return 0;
    constexpr int L = PRISM_RGLRU_CHUNK;
    const int chunks = (longest + L - 1) / L;
    if (S > 65535 || chunks > 65535) return (int)cudaErrorInvalidValue;
    const int threads = 64;
    dim3 grid((C + threads - 1) / threads, chunks, S);
    int rc = (int)prism::launch_kernel(prism::rglru_chunk_kernel<L>, grid, dim3(threads), 0, stream, a, g, ag_stride,
                                       (const float*)state, seg_start, slots, C, ws, ws0);
    if (rc) return rc;
    if (out_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::rglru_apply_kernel<__nv_bfloat16, L>, grid, dim3(threads), 0, stream, a, g,
                                         ag_stride, y, y_stride, state, seg_start, slots, C, act, (const float*)ws,
                                         (const float*)ws0, (__nv_bfloat16*)out, out_stride);
    return (int)prism::launch_kernel(prism::rglru_apply_kernel<float, L>, grid, dim3(threads), 0, stream, a, g, ag_stride, y,
                                     y_stride, state, seg_start, slots, C, act, (const float*)ws, (const float*)ws0,
                                     (float*)out, out_stride);
}
