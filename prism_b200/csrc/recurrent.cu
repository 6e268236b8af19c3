// Recurrent mixers: layers whose memory of a sequence is a matrix of fixed size per head instead of a cache of
// keys.  Two recurrences share one scan kernel; S is [dk, dv] per head, float32, one per request slot:
//
//   delta rule with a scalar decay (SCAN_DELTA), per token with unit-length q, k and g, beta in (0, 1):
//       S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees this token's write)
//   delta rule with one decay per key channel (SCAN_CHANNEL), w a vector over the key channels:
//       S <- diag(w) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//   decayed outer-product sum with a bonus for the current token (SCAN_BONUS), w, u vectors over the key channels:
//       o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T                    (the read-out sees S before the write)
//   generalized delta rule (SCAN_GENERAL), w, e, c vectors over the key channels (e the unit key, c = a * e a removal
//   rate per channel times it):
//       S <- diag(w) S - c (e^T S) + k v^T;   o = S^T r         (decay and removal both read the state before the token)
//
// Everything that enters the recurrence is float32: the kernels here read the float32 results of the input
// projections, and the state never leaves float32.  A request's state lives in its slot between steps, so
// the result at a position does not depend on how the request was cut into steps: the scan visits the
// tokens one after another either way, and the order of additions inside a token depends on the sizes only.
//
// Around the scans:
//   * prism_conv_unit_gates  per token: the short causal convolution over time of the q | k | v channels (its
//     last taps - 1 inputs per request are state too) with silu, q and k made unit vectors per head (q also
//     times dk^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias));
//   * prism_state_tail       the last rows of a step's input per request into a [slots, rows, width] state (the
//     convolution's tail; with one row, the previous token's input of a token-shift mix);
//   * prism_shift_mix        x + (x_prev - x) mu_s for several mu at once (x_prev of a step's first token comes
//     from the state);
//   * prism_headnorm_gate    o / rms(o) per head, times a weight, times silu(gate), times a constant.
#include "mma_helpers.cuh"

#define PRISM_SCAN_DELTA 0
#define PRISM_SCAN_BONUS 1
#define PRISM_SCAN_CHANNEL 2
#define PRISM_SCAN_GENERAL 3

namespace prism {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------------------------
// conv + silu, unit vectors, gates.  One CTA per token.
//   proj   [T, *] float32, row stride ps: columns [0, C) are the q | k | v channels (C = 2 G dk + H dv),
//          columns ob .. ob + H the beta projection, oa .. oa + H the decay projection
//   taps   [C, K] (last column: the current token's)
//   tail   [slots, K - 1, C] float32: the K - 1 inputs before the step's first token, oldest first
//   qkv    [T, C] float32 out;   bg [T, 2 H] float32 out: beta | g
// ---------------------------------------------------------------------------------------------------------
__global__ void conv_unit_gates_kernel(const float* __restrict__ proj_in, long long ps, int ob, int oa,
                                       const void* __restrict__ taps, int taps_bf16, int K,
                                       const float* tail, const void* __restrict__ a_log, int a_log_bf16,
                                       const void* __restrict__ dt_bias, int dt_bf16, const int* __restrict__ tok_seg,
                                       const int* __restrict__ seg_start, const int* __restrict__ slots, int G, int H,
                                       int dk, int dv, float unit_eps, float* __restrict__ qkv, float* __restrict__ bg,
                                       int move_tail) {
    pdl_trigger();
    pdl_wait();
    const float* proj = pdl_fresh(proj_in);
    extern __shared__ float y[];                       // [C]
    const int t = blockIdx.x, seg = tok_seg[t];
    const int i = t - seg_start[seg];                  // place of the token in its segment
    const int C = 2 * G * dk + H * dv;
    float* tl = const_cast<float*>(tail) + (size_t)slots[seg] * (K - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = K - 1; j >= 0; --j) {             // lag j: the input j tokens back; oldest first
            const int src = i - j;
            const float x = src >= 0 ? proj[(size_t)(t - j) * ps + c] : tl[(size_t)(K - 1 + src) * C + c];
            acc += load_param(taps, taps_bf16, (size_t)c * K + (K - 1 - j)) * x;
        }
        y[c] = silu_f(acc);
        // a step of single tokens: this CTA is the only reader of its request's tail, and a thread the only one of
        // its channel, so it moves the tail up by this token itself (no second launch)
        if (move_tail && K > 1) {
            for (int r = 0; r + 2 < K; ++r) tl[(size_t)r * C + c] = tl[(size_t)(r + 1) * C + c];
            tl[(size_t)(K - 2) * C + c] = proj[(size_t)t * ps + c];
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* out = qkv + (size_t)t * C;
    for (int hh = warp; hh < 2 * G; hh += nwarps) {    // q heads, then k heads
        const float* row = y + hh * dk;
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss += row[d] * row[d];
        ss = warp_sum(ss);
        const float inv = (1.f / sqrtf(ss + unit_eps)) * (hh < G ? 1.f / sqrtf((float)dk) : 1.f);
        for (int d = lane; d < dk; d += 32) out[hh * dk + d] = row[d] * inv;
    }
    for (int c = 2 * G * dk + threadIdx.x; c < C; c += blockDim.x) out[c] = y[c];
    if (a_log == nullptr) {            // the decay is formed elsewhere (one per key channel): bg [T, H] holds beta alone
        for (int h = threadIdx.x; h < H; h += blockDim.x) bg[(size_t)t * H + h] = sigmoid_f(proj[(size_t)t * ps + ob + h]);
        return;
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        bg[(size_t)t * 2 * H + h] = sigmoid_f(proj[(size_t)t * ps + ob + h]);
        const float dt = softplus_f(proj[(size_t)t * ps + oa + h] + load_param(dt_bias, dt_bf16, h));
        bg[(size_t)t * 2 * H + H + h] = expf(-expf(load_param(a_log, a_log_bf16, h)) * dt);
    }
}

// tail[slot][r][c] <- the input (rows - r) tokens before the end of the request's tokens so far: from this
// step's rows where the step reaches that far back, else from the tail as it was (shifted).  One CTA per
// segment; a thread owns a column, and walks r upwards, so that what it still needs is never overwritten.
__global__ void state_tail_kernel(const float* __restrict__ src_in, long long ss, int width, float* __restrict__ tail,
                                  int rows, const int* __restrict__ seg_start, const int* __restrict__ slots) {
    pdl_trigger();
    pdl_wait();
    const float* src = pdl_fresh(src_in);
    const int seg = blockIdx.x, s0 = seg_start[seg], qlen = seg_start[seg + 1] - s0;
    float* tl = tail + (size_t)slots[seg] * rows * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        for (int r = 0; r < rows; ++r) {
            const int idx = qlen - rows + r;           // place in the segment of the token that row r holds afterwards
            tl[(size_t)r * width + c] = idx >= 0 ? src[(size_t)(s0 + idx) * ss + c] : tl[(size_t)(r + qlen) * width + c];
        }
}

// out[s][t][c] = x[t][c] + (x_prev[t][c] - x[t][c]) mu[s][c],  s < n;  x_prev of a segment's first token is prev[slot].
template <typename T>
__global__ void shift_mix_kernel(const float* __restrict__ x_in, int D, const float* prev,
                                 const void* __restrict__ mu, int mu_bf16, int n, const int* __restrict__ tok_seg,
                                 const int* __restrict__ seg_start, const int* __restrict__ slots, T* __restrict__ out,
                                 long long out_plane, int keep_prev) {
    pdl_trigger();
    pdl_wait();
    const float* x = pdl_fresh(x_in);
    const int t = blockIdx.x, seg = tok_seg[t];
    float* own = const_cast<float*>(prev) + (size_t)slots[seg] * D;
    const float* xp = t > seg_start[seg] ? x + (size_t)(t - 1) * D : own;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float a = x[(size_t)t * D + c], d = xp[c] - a;
        for (int s = 0; s < n; ++s)
            out[(size_t)s * out_plane + (size_t)t * D + c] = from_float<T>(a + d * load_param(mu, mu_bf16, (size_t)s * D + c));
        if (keep_prev) own[c] = a;       // a step of single tokens: this token is its request's previous one from now on
    }
}

// w[t][c] <- exp(-exp(w[t][c] + w0[c])) in place: the decay of every key channel from its exponent, once for all
// the CTAs of the scan that read it (a step with many tokens; a decode step lets the scan do it).
__global__ void decay_from_exponent_kernel(float* __restrict__ w, long long ws, const void* __restrict__ w0, int w0_bf16, int A) {
    pdl_trigger();
    pdl_wait();
    float* row = pdl_fresh(w) + (size_t)blockIdx.y * ws;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < A; c += gridDim.x * blockDim.x)
        row[c] = expf(-expf(row[c] + load_param(w0, w0_bf16, c)));
}

// out[t][n] = epi(sum_r inner(low[t][r]) w2t[r][n] + b[n]): the second half of a low-rank product with what follows it,
// in one launch and float32 throughout.  inner: tanh (1) or nothing (0).  epi:
//   PRISM_LR_EXPEXP    exp(-exp(z))                          a per-channel decay from its double exponent
//   PRISM_LR_SOFTPLUS  exp(-exp(alog[n / per]) softplus(z))  a per-channel decay with one rate per group of `per` channels
//   PRISM_LR_SIGMOID   sigmoid(z)                            a gate
//   PRISM_LR_EXPSIG    exp(-rate sigmoid(z))                 a per-channel decay kept inside (exp(-rate), 1), rate a constant
// b may be null.  A CTA takes 128 channels and sixteen tokens, so that every weight it reads serves sixteen tokens
// (whose inner values sit side by side in shared memory: four 128-bit loads per weight); w2t is the second matrix
// transposed, [R, N], so that neighbouring threads read neighbouring floats.
#define PRISM_LR_EXPEXP 0
#define PRISM_LR_SOFTPLUS 1
#define PRISM_LR_SIGMOID 2
#define PRISM_LR_EXPSIG 3
constexpr int LRD_TOK = 16;
__global__ void lowrank_decay_kernel(const float* __restrict__ low_in, long long ls, int R, const float* __restrict__ w2t,
                                     const void* __restrict__ w0, int w0_bf16, int N, int T, float* __restrict__ out,
                                     long long os, int inner, int epi, const void* __restrict__ alog, int alog_bf16, int per,
                                     float crate) {
    pdl_trigger();
    pdl_wait();
    const float* low = pdl_fresh(low_in);
    extern __shared__ __align__(16) float s[];         // [R][LRD_TOK]
    const int t0 = blockIdx.y * LRD_TOK, n = blockIdx.x * blockDim.x + threadIdx.x;
    for (int i = threadIdx.x; i < LRD_TOK * R; i += blockDim.x) {
        const int j = i / R, r = i - j * R;            // neighbouring threads read neighbouring entries of a token's row
        const float v = t0 + j < T ? low[(size_t)(t0 + j) * ls + r] : 0.f;
        s[r * LRD_TOK + j] = inner ? tanhf(v) : v;
    }
    __syncthreads();
    if (n >= N) return;
    float acc[LRD_TOK];
#pragma unroll
    for (int j = 0; j < LRD_TOK; ++j) acc[j] = 0.f;
    for (int r = 0; r < R; ++r) {
        const float w = w2t[(size_t)r * N + n];
#pragma unroll
        for (int j = 0; j < LRD_TOK; j += 4) {
            const float4 t4 = *reinterpret_cast<const float4*>(s + r * LRD_TOK + j);
            acc[j] += w * t4.x;
            acc[j + 1] += w * t4.y;
            acc[j + 2] += w * t4.z;
            acc[j + 3] += w * t4.w;
        }
    }
    const float b = w0 != nullptr ? load_param(w0, w0_bf16, n) : 0.f;
    const float rate = epi == PRISM_LR_SOFTPLUS ? expf(load_param(alog, alog_bf16, n / per)) : 0.f;
#pragma unroll
    for (int j = 0; j < LRD_TOK; ++j)
        if (t0 + j < T) {
            const float z = acc[j] + b;
            out[(size_t)(t0 + j) * os + n] = epi == PRISM_LR_EXPEXP ? expf(-expf(z))
                                             : epi == PRISM_LR_SOFTPLUS ? expf(-rate * softplus_f(z))
                                             : epi == PRISM_LR_EXPSIG ? expf(-crate * sigmoid_f(z)) : sigmoid_f(z);
        }
}

// ex[t][h dk + i] = e_i = k_i / sqrt(sum_i k_i^2 + unit_eps) per head (the unit key), and
// ex[t][(H + h) dk + i] = sigmoid(a_i + ab[h dk + i]) e_i (the removal rate per channel times it): what the generalized
// delta rule takes out of its state.  k, a: float32 column blocks of one product (row stride ps).  One warp per (token, head).
__global__ void unit_removal_kernel(const float* __restrict__ k_in, const float* __restrict__ a_in, long long ps,
                                    const void* __restrict__ ab, int ab_bf16, float unit_eps, int Ttot, int H, int dk,
                                    float* __restrict__ ex) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)Ttot * H) return;
    const int t = (int)(w / H), h = (int)(w % H);
    const float* k = pdl_fresh(k_in) + (size_t)t * ps + (size_t)h * dk;
    const float* a = pdl_fresh(a_in) + (size_t)t * ps + (size_t)h * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += k[i] * k[i];
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss + unit_eps);
    float* e = ex + (size_t)t * 2 * H * dk + (size_t)h * dk;
    for (int i = lane; i < dk; i += 32) {
        const float u = k[i] * inv;
        e[i] = u;
        e[(size_t)H * dk + i] = sigmoid_f(a[i] + (ab != nullptr ? load_param(ab, ab_bf16, (size_t)h * dk + i) : 0.f)) * u;
    }
}

// out[t][h dv + c] = o[t][h][c] / sqrt(mean_c(o[t][h]^2) + eps) * weight[widx] * act(gate[t][h dv + c]) * scale,
// act silu, or sigmoid (gate_sigmoid; the gate may then hold the sigmoid already: gate_sigmoid 2),
// widx = c (one weight for all heads) or h dv + c (per_head_weight).  One warp per (token, head).
template <typename T>
__global__ void headnorm_gate_kernel(const float* __restrict__ o_in, const float* __restrict__ gate_in, long long gs,
                                     const void* __restrict__ weight, int weight_bf16, int per_head_weight, float eps,
                                     float scale, int Ttot, int H, int dv, T* __restrict__ out, long long os, int gate_sigmoid) {
    pdl_trigger();
    pdl_wait();
    const float* o = pdl_fresh(o_in);
    const float* gate = pdl_fresh(gate_in);
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)Ttot * H) return;
    const int t = (int)(w / H), h = (int)(w % H);
    const float* row = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss += row[c] * row[c];
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        const float wv = load_param(weight, weight_bf16, per_head_weight ? (size_t)h * dv + c : (size_t)c);
        const float gz = gate[(size_t)t * gs + (size_t)h * dv + c];
        const float g = gate_sigmoid == 2 ? gz : (gate_sigmoid ? sigmoid_f(gz) : silu_f(gz));
        out[(size_t)t * os + (size_t)h * dv + c] = from_float<T>(row[c] * inv * wv * g * scale);
    }
}

// ---------------------------------------------------------------------------------------------------------
// The scan.  grid (heads, segments, column blocks); the L threads of a column are neighbouring lanes of a warp,
// each owns R rows of that column of S in registers - quads of four neighbouring rows, quad part + L m - and
// they add up their partial dot products by shuffles.  The step's vectors come through shared memory TB tokens
// at a time with cp.async, the next block on its way while this one is worked on; a thread reads its quads
// of q, k (w, u) with 128-bit loads.  The state is kept in memory as [slot][head][column][row], so that the
// threads of a column read neighbouring floats.
//   SCAN_DELTA:  x [T, *] row stride xs: q of kv head g at qo + g dk, k at ko + g dk; v at vo + h dv;
//                bg [T, 2 H]: beta | g.
//   SCAN_BONUS:  r at qo + h dk, k at ko + h dk, v at vo + h dv, the decay's exponent ww [T, H dk] (row stride ws)
//                with w = exp(-exp(ww + w0)) formed in shared memory, w0 [H dk], bonus u [H dk].
//   SCAN_CHANNEL: q, k, v as for SCAN_DELTA; the decay itself in ww [T, H dk] (row stride ws); bg [T, H]: beta.
//   SCAN_GENERAL: r, k, v as for SCAN_BONUS; the decay itself in ww; ex [T, 2 H dk]: the unit key e at h dk, c at (H + h) dk.
// ---------------------------------------------------------------------------------------------------------
struct ScanArgs {
    const float* x;          // q | k | v (or r | k | v) rows
    long long xs;
    long long qo, ko, vo;
    const float* bg;         // DELTA: beta | g
    const float* ww;         // BONUS: the decay's exponent before w0
    long long ws;
    const void* w0;
    int w0_bf16;
    const void* u;
    int u_bf16;
    const float* ex;         // GENERAL: unit key | removal rate times unit key, [T, 2 H dk] (row stride es)
    long long es;
    float* state;            // [slots, H, dv, dk]
    const int* seg_start;
    const int* slots;
    float* out;              // [T, H, dv]
    int H, rep, dk, dkp, dv, cols, colsp, L, TB;
    int vec;                 // every source row piece starts on 16 bytes and is whole quads long
    int w_ready;             // BONUS: ww holds the decay itself already (prism_decay_from_exponent)
};

__device__ __forceinline__ void cp_async_f(float* smem, const float* gmem, int floats) {      // 1 or 4 floats
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    if (floats == 4) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem));
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem));
}

// sum over the L (a power of two, known when the kernel is compiled) neighbouring lanes that share a column
template <int L> __device__ __forceinline__ float column_sum(float v) {
    if (L > 16) v += __shfl_xor_sync(0xffffffffu, v, 16);
    if (L > 8) v += __shfl_xor_sync(0xffffffffu, v, 8);
    if (L > 4) v += __shfl_xor_sync(0xffffffffu, v, 4);
    if (L > 2) v += __shfl_xor_sync(0xffffffffu, v, 2);
    if (L > 1) v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

template <int MODE, int R, int L>
__global__ void scan_kernel(const ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int NV = MODE == PRISM_SCAN_DELTA ? 2 : (MODE == PRISM_SCAN_GENERAL ? 5 : 3);       // vectors over the key channels per token
    constexpr int Q = R / 4;                                   // quads of rows a thread owns
    const int h = blockIdx.x, seg = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int s0 = a.seg_start[seg], qlen = a.seg_start[seg + 1] - s0;
    const int dk = a.dk, dv = a.dv, TB = a.TB;
    constexpr int dkp = L * R;                                 // the rows a column's threads cover; beyond dk: zeros
    const int ncols = min(a.cols, dv - col0);
    // The CTA's last warp brings the step's vectors in (and, for the decayed sum, turns the decay's exponent into
    // the decay); the warps before it own the state.  Their threads beyond the CTA's columns run along (they
    // take part in the shuffles) and neither load nor store.
    const int CT = blockDim.x - 32;
    const bool producer = (int)threadIdx.x >= CT;
    const int part = threadIdx.x % L;
    const bool live = !producer && (int)threadIdx.x / L < ncols;
    const int lc = live ? threadIdx.x / L : 0, col = col0 + lc;
    const int kvh = h / a.rep;                         // DELTA: the q/k head this head uses
    // shared, per token of a block:  first[dkp] (q or r) | second[dkp] (k) | third[dkp] (BONUS: w) | v[colsp] | 4 scalars
    const int per_tok = NV * dkp + a.colsp + 4;
    constexpr int NBUF = 3;                            // blocks of tokens in shared memory: in use, landed, on its way
    float* ub = sm + (size_t)NBUF * TB * per_tok;      // BONUS: u[dkp]
    const float* x = pdl_fresh(a.x);
    const float* bg = pdl_fresh(a.bg);
    const float* ww = pdl_fresh(a.ww);
    const float* ex = pdl_fresh(a.ex);

    // padding entries of the staging buffers (rows beyond dk that the column's threads cover, columns beyond the
    // CTA's) are never written by the copies: zero them once
    if (dkp > dk || a.colsp > ncols) {
        const int pad = NV * (dkp - dk) + (a.colsp - ncols);
        for (int i = threadIdx.x; i < NBUF * TB * pad; i += blockDim.x) {
            const int slot = i / pad, c = i - slot * pad;
            const int which = c / (dkp - dk > 0 ? dkp - dk : 1);
            const int at = (dkp > dk && which < NV) ? which * dkp + dk + (c - which * (dkp - dk))
                                                    : NV * dkp + ncols + (c - NV * (dkp - dk));
            sm[(size_t)slot * per_tok + at] = 0.f;
        }
    }
    if (MODE == PRISM_SCAN_BONUS)
        for (int i = threadIdx.x; i < dkp; i += blockDim.x) ub[i] = i < dk ? load_param(a.u, a.u_bf16, (size_t)h * dk + i) : 0.f;
    __syncthreads();

    // the producer warp asks for block b0 of the segment's tokens into buffer `buf` ...
    auto stage = [&](int b0, int buf) {
        const int lane = threadIdx.x - CT;
        const int nb = min(TB, qlen - b0);
        float* dst0 = sm + (size_t)buf * TB * per_tok;
        const int unit = a.vec ? 4 : 1;
        const int nk = (dk + unit - 1) / unit, nc = (ncols + unit - 1) / unit;     // pieces per vector
        const size_t head_q = (size_t)((MODE == PRISM_SCAN_BONUS || MODE == PRISM_SCAN_GENERAL) ? h : kvh) * dk;
        for (int tt = 0; tt < nb; ++tt) {
            const size_t t = (size_t)(s0 + b0 + tt);
            const float* xr = x + t * a.xs;
            float* dst = dst0 + (size_t)tt * per_tok;
            for (int c = lane; c < nk; c += 32) {
                cp_async_f(dst + c * unit, xr + a.qo + head_q + c * unit, unit);
                cp_async_f(dst + dkp + c * unit, xr + a.ko + head_q + c * unit, unit);
                if (MODE != PRISM_SCAN_DELTA) cp_async_f(dst + 2 * dkp + c * unit, ww + t * a.ws + (size_t)h * dk + c * unit, unit);
                if (MODE == PRISM_SCAN_GENERAL) {
                    cp_async_f(dst + 3 * dkp + c * unit, ex + t * a.es + (size_t)h * dk + c * unit, unit);
                    cp_async_f(dst + 4 * dkp + c * unit, ex + t * a.es + (size_t)(a.H + h) * dk + c * unit, unit);
                }
            }
            for (int c = lane; c < nc; c += 32)
                cp_async_f(dst + NV * dkp + c * unit, xr + a.vo + (size_t)h * dv + col0 + c * unit, unit);
            if (MODE == PRISM_SCAN_DELTA && lane < 2)                                // beta, then g
                cp_async_f(dst + NV * dkp + a.colsp + lane, bg + t * 2 * a.H + (size_t)lane * a.H + h, 1);
            if (MODE == PRISM_SCAN_CHANNEL && lane == 0)                             // beta
                cp_async_f(dst + NV * dkp + a.colsp, bg + t * a.H + h, 1);
        }
        cp_async_commit();
    };
    // ... and, once the copies of that block have landed (the caller has waited), turns the decay's exponent into the decay
    auto finish = [&](int b0, int buf) {
        const int lane = threadIdx.x - CT;
        const int nb = min(TB, qlen - b0);
        float* dst0 = sm + (size_t)buf * TB * per_tok;
        __syncwarp();
        if (MODE == PRISM_SCAN_BONUS && !a.w_ready) {
            for (int idx = lane; idx < nb * dk; idx += 32) {
                const int tt = idx / dk, i = idx - tt * dk;
                float* w = dst0 + (size_t)tt * per_tok + 2 * dkp + i;
                *w = expf(-expf(*w + load_param(a.w0, a.w0_bf16, (size_t)h * dk + i)));
            }
        }
    };

    float S[R];
    float* st = a.state + (((size_t)a.slots[seg] * a.H + h) * dv + col) * dk;
    if (producer) {
        stage(0, 0);
        if (TB < qlen) stage(TB, 1);
        else cp_async_commit();
        cp_async_wait<1>();
        finish(0, 0);
    } else {
#pragma unroll
        for (int m = 0; m < Q; ++m) {
            const int i = 4 * (part + L * m);
            if (live && a.vec && i + 3 < dk) {
                const float4 v = *reinterpret_cast<const float4*>(st + i);
                S[4 * m] = v.x; S[4 * m + 1] = v.y; S[4 * m + 2] = v.z; S[4 * m + 3] = v.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) S[4 * m + j] = (live && i + j < dk) ? st[i + j] : 0.f;
            }
        }
    }
    __syncthreads();

    int buf = 0;
    for (int b0 = 0; b0 < qlen; b0 += TB, buf = buf + 1 == NBUF ? 0 : buf + 1) {
        const int nb = min(TB, qlen - b0);
        if (producer) {
            // while block b0 is worked on: ask for the block after the next (its buffer was freed at the last
            // barrier), and see the next one in
            const int nxt = buf + 1 == NBUF ? 0 : buf + 1, nxt2 = nxt + 1 == NBUF ? 0 : nxt + 1;
            if (b0 + 2 * TB < qlen) stage(b0 + 2 * TB, nxt2);
            else cp_async_commit();
            cp_async_wait<1>();
            if (b0 + TB < qlen) finish(b0 + TB, nxt);
            __syncthreads();
            continue;
        }
        const float* blk = sm + (size_t)buf * TB * per_tok;
        for (int tt = 0; tt < nb; ++tt) {
            const float* f1 = blk + (size_t)tt * per_tok;          // q or r
            const float* f2 = f1 + dkp;                            // k
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;         // four chains of multiply-adds side by side
            if (MODE == PRISM_SCAN_DELTA) {
                const float* vv = f2 + dkp;
                const float beta = vv[a.colsp], g = vv[a.colsp + 1];
                float k0 = 0.f, k1 = 0.f, k2 = 0.f, k3 = 0.f;
                float4 kq[Q];
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    kq[m] = *reinterpret_cast<const float4*>(f2 + 4 * (part + L * m));
                    k0 += S[4 * m] * kq[m].x;
                    k1 += S[4 * m + 1] * kq[m].y;
                    k2 += S[4 * m + 2] * kq[m].z;
                    k3 += S[4 * m + 3] * kq[m].w;
                }
                float ks = (k0 + k1) + (k2 + k3);
                ks = column_sum<L>(ks);
                const float uu = beta * (vv[lc] - g * ks);
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    const float4 qq = *reinterpret_cast<const float4*>(f1 + 4 * (part + L * m));
                    S[4 * m] = g * S[4 * m] + kq[m].x * uu;
                    S[4 * m + 1] = g * S[4 * m + 1] + kq[m].y * uu;
                    S[4 * m + 2] = g * S[4 * m + 2] + kq[m].z * uu;
                    S[4 * m + 3] = g * S[4 * m + 3] + kq[m].w * uu;
                    o0 += S[4 * m] * qq.x;
                    o1 += S[4 * m + 1] * qq.y;
                    o2 += S[4 * m + 2] * qq.z;
                    o3 += S[4 * m + 3] * qq.w;
                }
            } else if (MODE == PRISM_SCAN_CHANNEL) {
                const float* wd = f2 + dkp;
                const float* vv = wd + dkp;
                const float beta = vv[a.colsp];
                float k0 = 0.f, k1 = 0.f, k2 = 0.f, k3 = 0.f;
                float4 kq[Q];
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    const int i = 4 * (part + L * m);
                    kq[m] = *reinterpret_cast<const float4*>(f2 + i);
                    const float4 w4 = *reinterpret_cast<const float4*>(wd + i);
                    S[4 * m] *= w4.x;
                    S[4 * m + 1] *= w4.y;
                    S[4 * m + 2] *= w4.z;
                    S[4 * m + 3] *= w4.w;
                    k0 += S[4 * m] * kq[m].x;
                    k1 += S[4 * m + 1] * kq[m].y;
                    k2 += S[4 * m + 2] * kq[m].z;
                    k3 += S[4 * m + 3] * kq[m].w;
                }
                float ks = (k0 + k1) + (k2 + k3);
                ks = column_sum<L>(ks);
                const float uu = beta * (vv[lc] - ks);
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    const float4 qq = *reinterpret_cast<const float4*>(f1 + 4 * (part + L * m));
                    S[4 * m] += kq[m].x * uu;
                    S[4 * m + 1] += kq[m].y * uu;
                    S[4 * m + 2] += kq[m].z * uu;
                    S[4 * m + 3] += kq[m].w * uu;
                    o0 += S[4 * m] * qq.x;
                    o1 += S[4 * m + 1] * qq.y;
                    o2 += S[4 * m + 2] * qq.z;
                    o3 += S[4 * m + 3] * qq.w;
                }
            } else if (MODE == PRISM_SCAN_GENERAL) {
                const float* wd = f2 + dkp;            // decay | unit key | removal times unit key | v
                const float* ue = wd + dkp;
                const float* ce = ue + dkp;
                const float v = ce[dkp + lc];
                float k0 = 0.f, k1 = 0.f, k2 = 0.f, k3 = 0.f;
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    const float4 e4 = *reinterpret_cast<const float4*>(ue + 4 * (part + L * m));
                    k0 += S[4 * m] * e4.x;
                    k1 += S[4 * m + 1] * e4.y;
                    k2 += S[4 * m + 2] * e4.z;
                    k3 += S[4 * m + 3] * e4.w;
                }
                float es = (k0 + k1) + (k2 + k3);
                es = column_sum<L>(es);                // e^T S of this column, from the state before the token
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    const int i = 4 * (part + L * m);
                    const float4 rr = *reinterpret_cast<const float4*>(f1 + i), kk = *reinterpret_cast<const float4*>(f2 + i);
                    const float4 w4 = *reinterpret_cast<const float4*>(wd + i), c4 = *reinterpret_cast<const float4*>(ce + i);
                    S[4 * m] = w4.x * S[4 * m] - c4.x * es + kk.x * v;
                    S[4 * m + 1] = w4.y * S[4 * m + 1] - c4.y * es + kk.y * v;
                    S[4 * m + 2] = w4.z * S[4 * m + 2] - c4.z * es + kk.z * v;
                    S[4 * m + 3] = w4.w * S[4 * m + 3] - c4.w * es + kk.w * v;
                    o0 += S[4 * m] * rr.x;
                    o1 += S[4 * m + 1] * rr.y;
                    o2 += S[4 * m + 2] * rr.z;
                    o3 += S[4 * m + 3] * rr.w;
                }
            } else {
                const float* wd = f2 + dkp;
                const float v = wd[dkp + lc];
#pragma unroll
                for (int m = 0; m < Q; ++m) {
                    const int i = 4 * (part + L * m);
                    const float4 rr = *reinterpret_cast<const float4*>(f1 + i), kk = *reinterpret_cast<const float4*>(f2 + i);
                    const float4 w4 = *reinterpret_cast<const float4*>(wd + i), u4 = *reinterpret_cast<const float4*>(ub + i);
                    const float kv0 = kk.x * v, kv1 = kk.y * v, kv2 = kk.z * v, kv3 = kk.w * v;
                    o0 += rr.x * (S[4 * m] + u4.x * kv0);
                    o1 += rr.y * (S[4 * m + 1] + u4.y * kv1);
                    o2 += rr.z * (S[4 * m + 2] + u4.z * kv2);
                    o3 += rr.w * (S[4 * m + 3] + u4.w * kv3);
                    S[4 * m] = w4.x * S[4 * m] + kv0;
                    S[4 * m + 1] = w4.y * S[4 * m + 1] + kv1;
                    S[4 * m + 2] = w4.z * S[4 * m + 2] + kv2;
                    S[4 * m + 3] = w4.w * S[4 * m + 3] + kv3;
                }
            }
            float o = (o0 + o1) + (o2 + o3);
            o = column_sum<L>(o);
            if (live && part == 0) a.out[((size_t)(s0 + b0 + tt) * a.H + h) * dv + col] = o;
        }
        __syncthreads();                               // the next block has landed, and this buffer is free
    }
    if (live) {
#pragma unroll
        for (int m = 0; m < Q; ++m) {
            const int i = 4 * (part + L * m);
            if (a.vec && i + 3 < dk) {
                *reinterpret_cast<float4*>(st + i) = make_float4(S[4 * m], S[4 * m + 1], S[4 * m + 2], S[4 * m + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (i + j < dk) st[i + j] = S[4 * m + j];
            }
        }
    }
}

template <int MODE, int R, int L>
static int launch_scan(const ScanArgs& a, int S, cudaStream_t stream) {
    const int per_tok = (MODE == PRISM_SCAN_DELTA ? 2 : (MODE == PRISM_SCAN_GENERAL ? 5 : 3)) * a.dkp + a.colsp + 4;
    const size_t smem = ((size_t)3 * a.TB * per_tok + (MODE == PRISM_SCAN_BONUS ? a.dkp : 0)) * sizeof(float);
    auto kern = scan_kernel<MODE, R, L>;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(a.H, S, (a.dv + a.cols - 1) / a.cols);
    return (int)launch_kernel(kern, grid, dim3((a.cols * a.L + 31) / 32 * 32 + 32), smem, stream, a);      // + the producer warp
}

}  // namespace prism

PRISM_EXPORT int prism_conv_unit_gates(const float* proj, long long ps, int ob, int oa, const void* taps, int taps_dtype,
                                       int K, const float* tail, const void* a_log, int a_log_dtype, const void* dt_bias,
                                       int dt_dtype, const int* tok_seg, const int* seg_start, const int* slots, int T, int G,
                                       int H, int dk, int dv, float unit_eps, float* qkv, float* bg, int move_tail,
                                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (K < 1 || G < 1 || H < 1 || dk < 1 || dv < 1) return (int)cudaErrorInvalidValue;
    const int C = 2 * G * dk + H * dv;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kern = prism::conv_unit_gates_kernel;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int threads = C >= 2048 ? 1024 : (C >= 512 ? 256 : 128);          // a few channels a thread: their loads are one chain each
    return (int)prism::launch_kernel(kern, dim3(T), dim3(threads), smem, stream, proj, ps, ob, oa, taps,
                                     taps_dtype == PRISM_DTYPE_BF16, K, tail, a_log, a_log_dtype == PRISM_DTYPE_BF16, dt_bias,
                                     dt_dtype == PRISM_DTYPE_BF16, tok_seg, seg_start, slots, G, H, dk, dv, unit_eps, qkv, bg,
                                     move_tail);
}

PRISM_EXPORT int prism_state_tail(const float* src, long long src_stride, int width, float* tail, int rows,
                                  const int* seg_start, const int* slots, int S, cudaStream_t stream) {
    if (S <= 0 || rows <= 0 || width <= 0) return 0;
    return (int)prism::launch_kernel(prism::state_tail_kernel, dim3(S), dim3(width >= 1024 ? 256 : 128), 0, stream, src,
                                     src_stride, width, tail, rows, seg_start, slots);
}

PRISM_EXPORT int prism_shift_mix(const float* x, int D, const float* prev, const void* mu, int mu_dtype, int n,
                                 const int* tok_seg, const int* seg_start, const int* slots, int T, void* out, int out_dtype,
                                 long long out_plane, int keep_prev, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const int threads = D >= 2048 ? 1024 : (D >= 512 ? 256 : 128);
    const int mb = mu_dtype == PRISM_DTYPE_BF16;
    if (out_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::shift_mix_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, D, prev, mu,
                                         mb, n, tok_seg, seg_start, slots, (__nv_bfloat16*)out, out_plane, keep_prev);
    return (int)prism::launch_kernel(prism::shift_mix_kernel<float>, dim3(T), dim3(threads), 0, stream, x, D, prev, mu, mb, n,
                                     tok_seg, seg_start, slots, (float*)out, out_plane, keep_prev);
}

PRISM_EXPORT int prism_decay_from_exponent(float* w, long long w_stride, const void* w0, int w0_dtype, int T, int A,
                                           cudaStream_t stream) {
    if (T <= 0 || A <= 0) return 0;
    if (T > 65535) return (int)cudaErrorInvalidValue;
    return (int)prism::launch_kernel(prism::decay_from_exponent_kernel, dim3((A + 255) / 256, T), dim3(256), 0, stream, w,
                                     w_stride, w0, w0_dtype == PRISM_DTYPE_BF16, A);
}

// low [T, R] float32 (row stride free), w2t [R, N] float32, w0 [N] or null; out [T, N] float32; inner 1: tanh of low;
// epi PRISM_LR_*; alog [N / per] for PRISM_LR_SOFTPLUS; crate: the constant rate of PRISM_LR_EXPSIG.
PRISM_EXPORT int prism_lowrank_decay(const float* low, long long low_stride, int R, const float* w2t, const void* w0,
                                     int w0_dtype, int N, int T, float* out, long long out_stride, int inner, int epi,
                                     const void* alog, int alog_dtype, int per, float crate, cudaStream_t stream) {
    if (epi == PRISM_LR_SOFTPLUS && (alog == nullptr || per < 1)) return (int)cudaErrorInvalidValue;
    if (T <= 0 || N <= 0) return 0;
    const size_t smem = (size_t)prism::LRD_TOK * R * sizeof(float);
    if (R < 1 || smem > 200 * 1024 || (T + prism::LRD_TOK - 1) / prism::LRD_TOK > 65535) return (int)cudaErrorInvalidValue;
    auto kern = prism::lowrank_decay_kernel;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)prism::launch_kernel(kern, dim3((N + 127) / 128, (T + prism::LRD_TOK - 1) / prism::LRD_TOK), dim3(128), smem,
                                     stream, low, low_stride, R, w2t, w0, w0_dtype == PRISM_DTYPE_BF16, N, T, out, out_stride, inner, epi, alog,
                                     alog_dtype == PRISM_DTYPE_BF16, per < 1 ? 1 : per, crate);
}

// k, a [T, H dk] float32 column blocks with row stride ps; ab [H dk] or null; ex [T, 2 H dk] float32 out.
PRISM_EXPORT int prism_unit_removal(const float* k, const float* a, long long ps, const void* ab, int ab_dtype, float unit_eps,
                                    int T, int H, int dk, float* ex, cudaStream_t stream) {
    if (T <= 0 || H <= 0 || dk <= 0) return 0;
    const int warps = 4;
    const long long total = (long long)T * H;
    return (int)prism::launch_kernel(prism::unit_removal_kernel, dim3((unsigned)((total + warps - 1) / warps)), dim3(warps * 32), 0,
                                     stream, k, a, ps, ab, ab_dtype == PRISM_DTYPE_BF16, unit_eps, T, H, dk, ex);
}

PRISM_EXPORT int prism_headnorm_gate(const float* o, const float* gate, long long gate_stride, const void* weight,
                                     int weight_dtype, int per_head_weight, float eps, float scale, int T, int H, int dv,
                                     void* out, int out_dtype, long long out_stride, int gate_sigmoid, cudaStream_t stream) {
    if (T <= 0 || H <= 0 || dv <= 0) return 0;
    const int warps = 4;
    const long long total = (long long)T * H;
    const int blocks = (int)((total + warps - 1) / warps);
    const int wb = weight_dtype == PRISM_DTYPE_BF16;
    if (out_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::headnorm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, stream, o,
                                         gate, gate_stride, weight, wb, per_head_weight, eps, scale, T, H, dv,
                                         (__nv_bfloat16*)out, out_stride, gate_sigmoid);
    return (int)prism::launch_kernel(prism::headnorm_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, gate,
                                     gate_stride, weight, wb, per_head_weight, eps, scale, T, H, dv, (float*)out, out_stride, gate_sigmoid);
}

// mode PRISM_SCAN_*; state [slots, H, dv, dk] float32; out [T, H, dv] float32; rep: heads per q/k head (DELTA).
// Returns cudaErrorInvalidValue for dk > 1024.
PRISM_EXPORT int prism_recurrent_scan(int mode, const float* x, long long x_stride, long long qo, long long ko, long long vo,
                                      const float* bg,
                                      const float* ww, long long ww_stride, const void* w0, int w0_dtype, const void* u,
                                      int u_dtype, float* state, const int* seg_start, const int* slots, int S, int max_q_len,
                                      int H, int rep, int dk, int dv, float* out, int w_ready, const float* ex,
                                      long long ex_stride, cudaStream_t stream) {
    using namespace prism;
    if (S <= 0) return 0;
    if (H < 1 || rep < 1 || dk < 1 || dv < 1 || dk > 1024 || S > 65535) return (int)cudaErrorInvalidValue;
    ScanArgs a;
    a.x = x; a.xs = x_stride; a.qo = qo; a.ko = ko; a.vo = vo; a.bg = bg; a.ww = ww; a.ws = ww_stride;
    a.w0 = w0; a.w0_bf16 = w0_dtype == PRISM_DTYPE_BF16; a.u = u; a.u_bf16 = u_dtype == PRISM_DTYPE_BF16;
    a.state = state; a.seg_start = seg_start; a.slots = slots; a.out = out; a.H = H; a.rep = rep; a.dk = dk; a.dv = dv;
    a.w_ready = w_ready;
    a.ex = ex; a.es = ex_stride;
    if (mode == PRISM_SCAN_GENERAL && (ex == nullptr || ww == nullptr || rep != 1)) return (int)cudaErrorInvalidValue;
    // A token's work is one chain (dot product, shuffles, update, dot product, shuffles), so a CTA is latency
    // bound: eight threads a column, four warps of them side by side, and as many CTAs as there are column blocks.
    const int R = dk <= 32 ? 4 : (dk <= 64 ? 8 : (dk <= 128 ? 16 : 32));
    int L = 1;
    while (L * R < dk) L *= 2;                          // at most 32
    if (R >= 8 && L < 8) L = 8;                        // the compiled pairs: more than 32 rows always take eight threads a column
    a.L = L;
    a.dkp = L * R;                                     // the rows the threads of a column cover; beyond dk: zeros
    // 128 threads a CTA beside the producer warp; fewer (down to one warp) while the grid would leave SMs idle
    int threads = 128;
    while (threads > 32 && (long long)H * S * ((dv + threads / L - 1) / (threads / L)) < 148) threads /= 2;
    int cols = threads / L < 1 ? 1 : threads / L;
    if (cols > dv) cols = dv;
    if (cols >= 4) cols = cols / 4 * 4;
    a.cols = cols;
    a.colsp = (cols + 3) / 4 * 4;
    a.vec = dk % 4 == 0 && dv % 4 == 0 && cols % 4 == 0 && x_stride % 4 == 0 && qo % 4 == 0 && ko % 4 == 0 && vo % 4 == 0 &&
            (uintptr_t)x % 16 == 0 && (uintptr_t)state % 16 == 0 &&
            (mode == PRISM_SCAN_DELTA || (ww_stride % 4 == 0 && (uintptr_t)ww % 16 == 0)) &&
            (mode != PRISM_SCAN_GENERAL || (ex_stride % 4 == 0 && (uintptr_t)ex % 16 == 0 && ((long long)H * dk) % 4 == 0));
    const int per_tok = (mode == PRISM_SCAN_DELTA ? 2 : (mode == PRISM_SCAN_GENERAL ? 5 : 3)) * a.dkp + a.colsp + 4;
    int tb = (24 * 1024 / 4) / per_tok;
    tb = tb < 1 ? 1 : (tb > 16 ? 16 : tb);
    a.TB = tb > max_q_len ? (max_q_len < 1 ? 1 : max_q_len) : tb;      // a decode step stages one token, and CTAs are small
    // rows a thread and threads a column, both known to the compiler: (4, 1..8) up to 32 rows, (8, 8), (16, 8), (32, 8..32)
#define PRISM_SCAN(M)                                                                                \
    do {                                                                                             \
        if (R == 4) return L == 1 ? launch_scan<M, 4, 1>(a, S, stream) : L == 2 ? launch_scan<M, 4, 2>(a, S, stream)    \
                         : L == 4 ? launch_scan<M, 4, 4>(a, S, stream) : launch_scan<M, 4, 8>(a, S, stream);           \
        if (R == 8) return launch_scan<M, 8, 8>(a, S, stream);                                       \
        if (R == 16) return launch_scan<M, 16, 8>(a, S, stream);                                     \
        return L == 8 ? launch_scan<M, 32, 8>(a, S, stream) : L == 16 ? launch_scan<M, 32, 16>(a, S, stream)           \
                      : launch_scan<M, 32, 32>(a, S, stream);                                        \
    } while (0)
    if (mode == PRISM_SCAN_DELTA) PRISM_SCAN(PRISM_SCAN_DELTA);
    if (mode == PRISM_SCAN_BONUS) PRISM_SCAN(PRISM_SCAN_BONUS);
    if (mode == PRISM_SCAN_CHANNEL) PRISM_SCAN(PRISM_SCAN_CHANNEL);
    if (mode == PRISM_SCAN_GENERAL) PRISM_SCAN(PRISM_SCAN_GENERAL);
#undef PRISM_SCAN
    return (int)cudaErrorInvalidValue;
}
