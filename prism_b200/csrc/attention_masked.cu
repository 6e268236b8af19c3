// bf16 paged attention on tensor cores for layers that the equal-size causal kernels (attention_bf16.cu) do
// not cover: keys of dk and values of dv entries per head (dv != dk allowed, and the values may be the leading
// entries of the key rows themselves), a key mask of any PRISM_MASK_* kind, and an optional sink in the
// softmax's denominator, and an optional bias by distance (a float32 table [nh, dist_max + 1]: the key n positions
// back gets table[h][min(n, dist_max)] added to its scaled score).
//
// A CTA takes one segment, one kv head and 64 rows; a row is a (query token, query head of that kv head)
// pair, so the nh / nkv heads that share a kv head sit side by side and every key/value tile is read once
// for all of them (with one kv head - latent attention - all heads of a token share the tile).  Key tiles of
// 64 come through the block table with 16-byte cp.async, double-buffered.  Scores (m16n8k16 bf16 MMA, float32
// accumulation), the scale, the mask, running maximum and sum, and the normalisation are float32.  The
// softmax weights enter the PV product as two bf16 terms, hi = bf16(p) and lo = bf16(p - hi), so they carry
// 16 mantissa bits instead of 8: the weights are float32 quantities by the model's definition, and one
// rounding to bf16 would be the largest error of the layer.
//
// Two shapes of the same loop:
//   * portions (SPLITK false): warp w owns rows 16 w .. 16 w + 15 and walks all 64 keys of a tile;
//   * few rows (SPLITK true; a decode step: one token per segment; a CTA takes up to 16 of the heads of a kv
//     head): all four warps own the same 16 rows, warp w takes keys 16 w .. 16 w + 15 of every tile, and the
//     four partial (max, sum, output) are merged through shared memory at the end; several CTAs may share the
//     key tiles of one (segment, kv head), and a second kernel merges their partial results.
// The order of additions for a position depends on its place in the CTA's row tile, i.e. on how the request
// was cut into steps, only through float32 rounding.
#include <algorithm>

#include "mma_helpers.cuh"

namespace prism {

#ifndef PRISM_MA_PORTION_STAGES
#define PRISM_MA_PORTION_STAGES 2
#endif
#ifndef PRISM_MA_PORTION_TILE
#define PRISM_MA_PORTION_TILE 32
#endif
// keys per tile: 64 in the few-rows shape (16 for each warp); in the portions shape 32, which with two stages
// leaves room for three or four CTAs per SM instead of two
constexpr int MA_TILE_DECODE = 64;
constexpr int MA_TILE_PORTION = PRISM_MA_PORTION_TILE;
constexpr int MA_THREADS = 128;
constexpr int MA_ROWS = 64;

struct MaskedAttn {
    const __nv_bfloat16* q;
    long long q_stride;
    int q_head_stride;
    __nv_bfloat16* out;
    long long out_stride;
    const __nv_bfloat16* kc;
    long long k_row_stride;
    int k_head_stride;
    const __nv_bfloat16* vc;
    long long v_row_stride;
    int v_head_stride;
    const int* block_table;
    int bt_width;
    const int* seg_start;
    const int* cached_len;
    int nh, nkv, dk, dkp, dv, page_size, num_pages, mask_kind, mask_size;
    int mask_keep;     // under a window: the first mask_keep positions stay visible to every later query
    float scale_log2;
    const void* sink;
    int sink_bf16;
    int* err;
    int rpt;           // rows per token: the query heads of one kv head (at most 64 of them per CTA)
    int tok_per_cta;   // 64 / rpt
    int hgroups;       // CTAs that share the heads of one kv head when there are more than hrows
    int hrows;         // query heads of one kv head a CTA takes at most: 64, in the few-rows shape 16
    int page_shift;    // log2(page_size), or -1
    int nsplit;        // few-rows shape: CTAs that share one (segment, kv head)'s key tiles
    float* part_o;     // [segments, nh, nsplit, dv]   their partial outputs (not normalised) ...
    float* part_ml;    // [segments, nh, nsplit, 2]    ... with running maximum (log2 domain) and sum
    const float* dist_bias;   // [nh, dist_max + 1] or null: added to the scaled score of the key min(p - key, dist_max) back
    int dist_max;
};

__device__ __forceinline__ int ma_first_key(int kind, int size, int pos) {
    if (kind == PRISM_MASK_WINDOW) return pos - size + 1 > 0 ? pos - size + 1 : 0;
    if (kind == PRISM_MASK_CHUNK) return pos / size * size;
    return 0;
}

__device__ __forceinline__ float ma_exp2(float x) {      // 0 for -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ROWS (32 or 64) cache rows (keys first_key ..) of one kv head into ks[ROWS][kstride] and, unless the values are
// read out of the key rows, vs[ROWS][vstride].  A row is `kchunks` (`vchunks`) 16-byte pieces, of which the first `kreal`
// (`vreal`) come from the plane and the rest are zero; keys outside [lo, hi] (and not below `keep`) are zero rows.  Sixteen threads
// share a row and a thread serves rows tid / 16 + 8 j: it first looks up the slots of its eight rows (eight
// independent loads of the block table, in flight together), then issues the copies.
template <bool WITH_V, int ROWS>
__device__ __forceinline__ void ma_load_tile(__nv_bfloat16* ks, int kstride, int kchunks, int kreal,
                                             __nv_bfloat16* vs, int vstride, int vchunks, int vreal,
                                             const __nv_bfloat16* __restrict__ kplane, long long k_row_stride, size_t k_head_off,
                                             const __nv_bfloat16* __restrict__ vplane, long long v_row_stride, size_t v_head_off,
                                             const int* __restrict__ bt, int first_key, int lo, int hi, int keep,
                                             int page_size, int page_shift, int num_pages, int* err, int tid) {
    const int rr = tid >> 4, cc = tid & 15;
    constexpr int PASSES = ROWS / 8;
    long long slot[PASSES];
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
        const int key = first_key + rr + 8 * j;
        slot[j] = -1;
        if ((key >= lo || key < keep) && key <= hi) {
            const int page = page_shift >= 0 ? bt[key >> page_shift] : bt[key / page_size];
            const int in_page = page_shift >= 0 ? (key & (page_size - 1)) : key % page_size;
            if (page < 0 || page >= num_pages) report_error(err, PRISM_ERR_PAGE_RANGE);
            else slot[j] = (long long)page * page_size + in_page;
        }
    }
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
        const int r = rr + 8 * j;
        const bool row_ok = slot[j] >= 0;
        const __nv_bfloat16* ksrc = kplane + (row_ok ? (size_t)slot[j] * (size_t)k_row_stride + k_head_off : 0);
        for (int c = cc; c < kchunks; c += 16) {
            const bool v = row_ok && c < kreal;
            cp_async16(ks + r * kstride + c * 8, v ? ksrc + c * 8 : kplane, v);
        }
        if (WITH_V) {
            const __nv_bfloat16* vsrc = vplane + (row_ok ? (size_t)slot[j] * (size_t)v_row_stride + v_head_off : 0);
            for (int c = cc; c < vchunks; c += 16) {
                const bool v = row_ok && c < vreal;
                cp_async16(vs + r * vstride + c * 8, v ? vsrc + c * 8 : vplane, v);
            }
        }
    }
}

template <int DVP, bool V_IN_K, bool SPLITK>
__global__ void __launch_bounds__(MA_THREADS, (!SPLITK && DVP <= 128 && PRISM_MA_PORTION_TILE == 32) ? 3 : 1)
attn_masked_kernel(const MaskedAttn a) {
    pdl_trigger();
    pdl_wait();
    constexpr int MA_TILE = SPLITK ? MA_TILE_DECODE : MA_TILE_PORTION;
    constexpr int NT = SPLITK ? 2 : MA_TILE / 8;       // 8-key score tiles per warp and key tile
    constexpr int STAGES = SPLITK ? 3 : PRISM_MA_PORTION_STAGES;   // a decode CTA has little to compute: more tiles in flight
    constexpr int QROWS = SPLITK ? 16 : MA_ROWS;       // query rows the CTA keeps in shared memory
    const int seg = blockIdx.z;
    const int kvh = blockIdx.y / a.hgroups, hg = blockIdx.y % a.hgroups;
    const int s0 = a.seg_start[seg], qlen = a.seg_start[seg + 1] - s0;
    // later row tiles see more keys: they start first.  In the few-rows shape x counts the key splits instead.
    const int q0 = SPLITK ? 0 : (gridDim.x - 1 - blockIdx.x) * a.tok_per_cta;
    if (q0 >= qlen) return;
    const int ntok = min(a.tok_per_cta, qlen - q0);
    const int rep = a.nh / a.nkv;
    const int head0 = kvh * rep + hg * a.hrows;                           // head of a token's first row
    const int nheads = min(a.rpt, rep - hg * a.hrows);                    // rows of a token that are real
    const int pos0 = a.cached_len[seg] + q0;
    const int* bt = a.block_table + (size_t)seg * a.bt_width;

    const int kstride = a.dkp + 8, vstride = V_IN_K ? kstride : DVP + 8;
    const int k_elems = MA_TILE * kstride, v_elems = V_IN_K ? 0 : MA_TILE * vstride;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [QROWS][kstride]
    __nv_bfloat16* KV = Qs + QROWS * kstride;                                   // [stage][K | V]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lo = ma_first_key(a.mask_kind, a.mask_size, pos0);
    const int hi = pos0 + ntok - 1;
    // The key tiles this CTA walks: those that hold kept first positions and lie wholly before the window
    // (tiles 0 .. kt - 1), then the window's (tw0 ..).  v0 .. v1 - 1 counts through both runs.
    const int tw0 = lo / MA_TILE;
    const int kt = min((min(a.mask_keep, lo) + MA_TILE - 1) / MA_TILE, tw0);
    int v0 = 0, v1 = kt + hi / MA_TILE + 1 - tw0;
    if (SPLITK && a.nsplit > 1) {                      // this CTA's share of the key tiles (it may be empty)
        const int per = (v1 - v0 + a.nsplit - 1) / a.nsplit;
        v0 += blockIdx.x * per;
        v1 = min(v1, v0 + per);
    }
    auto tile_of = [&](int v) { return v < kt ? v : tw0 + (v - kt); };

    {   // the CTA's query rows
        const int chunks = a.dkp / 8, real = a.dk / 8;
        for (int i = tid; i < QROWS * chunks; i += MA_THREADS) {
            const int r = i / chunks, c = i - r * chunks;
            const int tk = r / a.rpt, hh = r - tk * a.rpt;
            const bool valid = tk < ntok && hh < nheads && c < real;
            const __nv_bfloat16* src = a.q;
            if (valid) src += (size_t)(s0 + q0 + tk) * a.q_stride + (size_t)(head0 + hh) * a.q_head_stride + c * 8;
            cp_async16(Qs + r * kstride + c * 8, src, valid);
        }
    }
    auto load_tile = [&](int tile, int stage) {
        __nv_bfloat16* ks = KV + (size_t)stage * (k_elems + v_elems);
        ma_load_tile<!V_IN_K, MA_TILE>(ks, kstride, a.dkp / 8, a.dk / 8, ks + k_elems, vstride, DVP / 8, (a.dv + 7) / 8, a.kc,
                              a.k_row_stride, (size_t)kvh * a.k_head_stride, a.vc, a.v_row_stride,
                              (size_t)kvh * a.v_head_stride, bt, tile * MA_TILE, lo, hi, a.mask_keep, a.page_size, a.page_shift,
                              a.num_pages, a.err, tid);
    };
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {           // the first group also holds the query rows
        if (v0 + st < v1) load_tile(tile_of(v0 + st), st);
        cp_async_commit();
    }

    float o[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int mat = lane >> 3, lr = lane & 7;
    const int rowbase = SPLITK ? 0 : warp * 16;
    const int keybase = SPLITK ? warp * 16 : 0;
    // the two rows this thread holds scores of
    int p_row[2], lo_row[2];
    bool ok_row[2];
    const float* bias_row[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = rowbase + (lane >> 2) + e * 8;
        const int tk = r / a.rpt, hh = r - tk * a.rpt;
        ok_row[e] = tk < ntok && hh < nheads;
        bias_row[e] = a.dist_bias != nullptr ? a.dist_bias + (size_t)(head0 + (hh < nheads ? hh : 0)) * (a.dist_max + 1) : nullptr;
        p_row[e] = pos0 + (tk < ntok ? tk : ntok - 1);
        lo_row[e] = ma_first_key(a.mask_kind, a.mask_size, p_row[e]);
    }
    // keys that any row of this warp sees
    const int w_tk0 = min(rowbase / a.rpt, ntok - 1), w_tk1 = min((rowbase + 15) / a.rpt, ntok - 1);
    const int w_lo = ma_first_key(a.mask_kind, a.mask_size, pos0 + w_tk0), w_hi = pos0 + w_tk1;
    const bool warp_has_rows = rowbase / a.rpt < ntok;
    const int w_lo_last = ma_first_key(a.mask_kind, a.mask_size, w_hi);          // the last row's first key: the largest
    const bool w_all_rows = (rowbase + 15) / a.rpt < ntok && nheads == a.rpt;    // all 16 rows are real

    for (int vt = v0; vt < v1; ++vt) {
        const int it = vt - v0, tile = tile_of(vt);
        if (vt + STAGES - 1 < v1) load_tile(tile_of(vt + STAGES - 1), (it + STAGES - 1) % STAGES);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const __nv_bfloat16* Ks = KV + (size_t)(it % STAGES) * (k_elems + v_elems);
        const __nv_bfloat16* Vs = V_IN_K ? Ks : Ks + k_elems;
        const int kfirst = tile * MA_TILE + keybase, klast = kfirst + NT * 8 - 1;
        if (warp_has_rows && kfirst <= w_hi && (klast >= w_lo || kfirst < a.mask_keep)) {
            float s[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            for (int ks = 0; ks < a.dkp / 16; ++ks) {
                uint32_t qa[4];
                ldmatrix_x4(qa, Qs + (rowbase + lr + (mat & 1) * 8) * kstride + ks * 16 + (mat >> 1) * 8);
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, Ks + (keybase + np * 16 + (mat >> 1) * 8 + lr) * kstride + ks * 16 + (mat & 1) * 8);
                    mma_bf16_16816(s[2 * np], qa, b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], qa, b[2], b[3]);
                }
            }
            const int key0 = kfirst + (lane & 3) * 2;
            float mx[2] = {-INFINITY, -INFINITY};
            // only a tile that crosses some row's first or last visible key (or a warp with unused rows) needs the mask
            if (a.dist_bias != nullptr || !w_all_rows || kfirst < w_lo_last || klast > pos0 + w_tk0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + nt * 8 + (e & 1);
                        const int rr = e >> 1;
                        const bool vis = ok_row[rr] && key <= p_row[rr] && (key >= lo_row[rr] || key < a.mask_keep);
                        float v = -INFINITY;
                        if (vis) {
                            v = s[nt][e] * a.scale_log2;
                            if (bias_row[rr] != nullptr) v += bias_row[rr][min(p_row[rr] - key, a.dist_max)] * 1.4426950408889634f;
                        }
                        s[nt][e] = v;
                        mx[rr] = fmaxf(mx[rr], v);
                    }
            } else {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = s[nt][e] * a.scale_log2;
                        s[nt][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
            }
            float corr[2], mu[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                mu[r] = m_new == -INFINITY ? 0.f : m_new;       // finite, so exp2(-inf - mu) = 0
                corr[r] = ma_exp2(m_run[r] - mu[r]);
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = ma_exp2(s[nt][e] - mu[e >> 1]);
                    s[nt][e] = p;
                    l_run[e >> 1] += p;
                }
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                uint32_t ph[4], pl[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float x0 = s[2 * kk + (u >> 1)][(u & 1) * 2], x1 = s[2 * kk + (u >> 1)][(u & 1) * 2 + 1];
                    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
                    const float2 hf = __bfloat1622float2(h);
                    ph[u] = *reinterpret_cast<const uint32_t*>(&h);
                    pl[u] = pack_bf16(x0 - hf.x, x1 - hf.y);
                }
#pragma unroll
                for (int j = 0; j < DVP / 16; ++j) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, Vs + (keybase + kk * 16 + (mat & 1) * 8 + lr) * vstride + j * 16 + (mat >> 1) * 8);
                    mma_bf16_16816(o[2 * j], ph, b[0], b[1]);
                    mma_bf16_16816(o[2 * j + 1], ph, b[2], b[3]);
                    mma_bf16_16816(o[2 * j], pl, b[0], b[1]);
                    mma_bf16_16816(o[2 * j + 1], pl, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    constexpr float LOG2E = 1.4426950408889634f;
    if (!SPLITK) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = rowbase + (lane >> 2) + e * 8;
            const int tk = r / a.rpt, hh = r - tk * a.rpt;
            if (!ok_row[e]) continue;
            float l = l_run[e], f = 1.f;
            if (a.sink != nullptr) {
                const float sk = load_param(a.sink, a.sink_bf16, head0 + hh) * LOG2E;
                const float m_all = fmaxf(m_run[e], sk);
                f = ma_exp2(m_run[e] - m_all);
                l = l * f + ma_exp2(sk - m_all);
            }
            const float inv = l > 0.f ? f / l : 0.f;
            __nv_bfloat16* orow = a.out + (size_t)(s0 + q0 + tk) * a.out_stride + (size_t)(head0 + hh) * a.dv;
#pragma unroll
            for (int nt = 0; nt < DVP / 8; ++nt) {
                const int d = nt * 8 + (lane & 3) * 2;
                if (d < a.dv)
                    *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16(o[nt][2 * e] * inv, o[nt][2 * e + 1] * inv);
            }
        }
        return;
    }
    // SPLITK: the four warps' partial results of the same 16 rows, merged through shared memory
    __syncthreads();             // every thread's copies have landed before the buffers are used for something else
    float* sm_o = reinterpret_cast<float*>(smem_raw);            // [4][16][DVP]
    float* sm_ml = sm_o + 4 * 16 * DVP;                          // [4][16][2]
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = (lane >> 2) + e * 8;
        if ((lane & 3) == 0) {
            sm_ml[(warp * 16 + r) * 2] = m_run[e];
            sm_ml[(warp * 16 + r) * 2 + 1] = l_run[e];
        }
#pragma unroll
        for (int nt = 0; nt < DVP / 8; ++nt) {
            const int d = nt * 8 + (lane & 3) * 2;
            sm_o[(warp * 16 + r) * DVP + d] = o[nt][2 * e];
            sm_o[(warp * 16 + r) * DVP + d + 1] = o[nt][2 * e + 1];
        }
    }
    __syncthreads();
    for (int i = tid; i < 16 * (DVP / 2); i += MA_THREADS) {
        const int r = i / (DVP / 2), d = (i - r * (DVP / 2)) * 2;
        const int tk = r / a.rpt, hh = r - tk * a.rpt;
        if (tk >= ntok || hh >= nheads || d >= a.dv) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        const bool last = a.nsplit <= 1;                 // no other CTA shares these keys: finish here, sink included
        if (last && a.sink != nullptr) M = fmaxf(M, load_param(a.sink, a.sink_bf16, head0 + hh) * LOG2E);
        const float Mu = M == -INFINITY ? 0.f : M;
        float L = 0.f, x0 = 0.f, x1 = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = ma_exp2(sm_ml[(w * 16 + r) * 2] - Mu);
            L += sm_ml[(w * 16 + r) * 2 + 1] * f;
            x0 += sm_o[(w * 16 + r) * DVP + d] * f;
            x1 += sm_o[(w * 16 + r) * DVP + d + 1] * f;
        }
        if (!last) {                                     // partial result of this CTA's keys, for the merge kernel
            const size_t slot = ((size_t)(s0 + tk) * a.nh + head0 + hh) * a.nsplit + blockIdx.x;
            a.part_o[slot * a.dv + d] = x0;
            a.part_o[slot * a.dv + d + 1] = x1;
            if (d == 0) {
                a.part_ml[slot * 2] = M;
                a.part_ml[slot * 2 + 1] = L;
            }
            continue;
        }
        if (a.sink != nullptr) L += ma_exp2(load_param(a.sink, a.sink_bf16, head0 + hh) * LOG2E - Mu);
        const float inv = L > 0.f ? 1.f / L : 0.f;
        __nv_bfloat16* orow = a.out + (size_t)(s0 + q0 + tk) * a.out_stride + (size_t)(head0 + hh) * a.dv;
        *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16(x0 * inv, x1 * inv);
    }
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / (sum_s l_s 2^(m_s - M) + 2^(sink_h - M)) over the key splits' partial results
__global__ void attn_masked_merge_kernel(const float* __restrict__ part_o_, const float* __restrict__ part_ml_, int nsplit,
                                         int dv, int nh, const void* __restrict__ sink, int sink_bf16,
                                         __nv_bfloat16* __restrict__ out, long long out_stride) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x / nh, h = blockIdx.x % nh;
    const float* po = pdl_fresh(part_o_) + (size_t)blockIdx.x * nsplit * dv;
    const float* pml = pdl_fresh(part_ml_) + (size_t)blockIdx.x * nsplit * 2;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, pml[2 * s]);
    const float sk = sink != nullptr ? load_param(sink, sink_bf16, h) * 1.4426950408889634f : -INFINITY;
    M = fmaxf(M, sk);
    const float Mu = M == -INFINITY ? 0.f : M;
    float L = ma_exp2(sk - Mu);
    for (int s = 0; s < nsplit; ++s) L += pml[2 * s + 1] * ma_exp2(pml[2 * s] - Mu);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < nsplit; ++s) acc += po[(size_t)s * dv + d] * ma_exp2(pml[2 * s] - Mu);
        out[(size_t)t * out_stride + (size_t)h * dv + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int DVP, bool V_IN_K, bool SPLITK>
static int launch_masked(const MaskedAttn& a, int S, int max_q_len, cudaStream_t stream) {
    const int kstride = a.dkp + 8, vstride = DVP + 8;
    // V_IN_K: the value fragments of the padded columns dv .. DVP - 1 (never stored) may be read past a key row's
    // end, for the last row of the last stage past the tile: DVP spare elements keep that inside the allocation
    constexpr int STAGES = SPLITK ? 3 : PRISM_MA_PORTION_STAGES;
    constexpr int MA_TILE = SPLITK ? MA_TILE_DECODE : MA_TILE_PORTION;
    size_t smem = (size_t)((SPLITK ? 16 : MA_ROWS) * kstride + STAGES * (MA_TILE * kstride + (V_IN_K ? 0 : MA_TILE * vstride)) + (V_IN_K ? DVP : 0)) *
                  sizeof(__nv_bfloat16);
    if (SPLITK) smem = std::max(smem, (size_t)(4 * 16 * DVP + 4 * 16 * 2) * sizeof(float));
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    auto kern = attn_masked_kernel<DVP, V_IN_K, SPLITK>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(SPLITK ? a.nsplit : (max_q_len + a.tok_per_cta - 1) / a.tok_per_cta, a.nkv * a.hgroups, S);
    const cudaError_t rc = launch_kernel(kern, grid, dim3(MA_THREADS), smem, stream, a);
    if (rc != cudaSuccess || !SPLITK || a.nsplit <= 1) return (int)rc;
    return (int)launch_kernel(attn_masked_merge_kernel, dim3(S * a.nh), dim3(a.dv >= 128 ? 128 : 64), 0, stream,
                              (const float*)a.part_o, (const float*)a.part_ml, a.nsplit, a.dv, a.nh, a.sink, a.sink_bf16,
                              a.out, a.out_stride);
}

}  // namespace prism

// Whether the tensor-core kernel takes these sizes: keys and values in whole 16-byte pieces, values up to
// 256 entries (the output tile lives in registers), keys up to 576.
PRISM_EXPORT int prism_attention_masked_supported(int dk, int dv, int nh, int nkv) {
    return dk >= 8 && dk % 8 == 0 && dk <= 576 && dv >= 2 && dv % 2 == 0 && dv <= 256 && nkv > 0 && nh % nkv == 0;
}

// q [T, nh, dk] bf16 (token and head strides in elements, multiples of 8); out [T, nh * dv]; planes as for
// prism_attention_masked_generic; vc == nullptr: the values are the first dv entries of the key rows.
// few_rows != 0: every segment has one token; then nsplit
// CTAs share the key tiles of one (segment, kv head), and for nsplit > 1 leave partial results in part_o
// [S, nh, nsplit, dv] and part_ml [S, nh, nsplit, 2] (float32) for a merge kernel.
PRISM_EXPORT int prism_attention_masked_bf16(const void* q, long long q_stride, int q_head_stride, void* out,
                                             long long out_stride, const void* kc, long long k_row_stride,
                                             int k_head_stride, const void* vc, long long v_row_stride,
                                             int v_head_stride, const int* block_table, int bt_width,
                                             const int* seg_start, const int* cached_len, int S, int max_q_len,
                                             int nh, int nkv, int dk, int dv, int page_size, int num_pages,
                                             int mask_kind, int mask_size, int mask_keep, float scale,
                                             const void* sink, int sink_dtype, int few_rows, int nsplit, float* part_o, float* part_ml,
                                             int* err, const float* dist_bias, int dist_max, cudaStream_t stream) {
    using namespace prism;
    if (S <= 0 || max_q_len <= 0) return 0;
    if (!prism_attention_masked_supported(dk, dv, nh, nkv)) return (int)cudaErrorInvalidValue;
    const bool v_in_k = vc == nullptr;
    if (q_stride % 8 || q_head_stride % 8 || k_row_stride % 8 || k_head_stride % 8 || (uintptr_t)q % 16 || (uintptr_t)kc % 16 ||
        (!v_in_k && (v_row_stride % 8 || v_head_stride % 8 || (uintptr_t)vc % 16 || dv % 8)) || (v_in_k && dv > dk) ||
        (mask_kind != PRISM_MASK_CAUSAL && mask_size < 1) || mask_keep < 0 || (mask_keep > 0 && mask_kind != PRISM_MASK_WINDOW))
        return (int)cudaErrorInvalidValue;
    const int rep = nh / nkv;
    if (few_rows && (max_q_len != 1 || nsplit < 1 || nsplit > 65535 ||
                     (nsplit > 1 && (part_o == nullptr || part_ml == nullptr))))
        return (int)cudaErrorInvalidValue;
    MaskedAttn a;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.q_head_stride = q_head_stride;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.kc = (const __nv_bfloat16*)kc; a.k_row_stride = k_row_stride; a.k_head_stride = k_head_stride;
    a.vc = (const __nv_bfloat16*)vc; a.v_row_stride = v_row_stride; a.v_head_stride = v_head_stride;
    a.block_table = block_table; a.bt_width = bt_width; a.seg_start = seg_start; a.cached_len = cached_len;
    a.nh = nh; a.nkv = nkv; a.dk = dk; a.dkp = (dk + 15) / 16 * 16; a.dv = dv; a.page_size = page_size;
    a.num_pages = num_pages; a.mask_kind = mask_kind; a.mask_size = mask_size; a.mask_keep = mask_keep;
    a.scale_log2 = scale * 1.4426950408889634f; a.sink = sink; a.sink_bf16 = sink_dtype == PRISM_DTYPE_BF16; a.err = err;
    a.hrows = few_rows ? 16 : MA_ROWS;
    a.rpt = rep < a.hrows ? rep : a.hrows;
    a.tok_per_cta = few_rows ? 1 : MA_ROWS / a.rpt;
    a.hgroups = (rep + a.hrows - 1) / a.hrows;
    a.page_shift = -1;
    if (page_size > 0 && (page_size & (page_size - 1)) == 0)
        for (a.page_shift = 0; (1 << a.page_shift) < page_size;) ++a.page_shift;
    a.nsplit = few_rows ? nsplit : 1;
    a.part_o = part_o;
    a.part_ml = part_ml;
    a.dist_bias = dist_bias;
    a.dist_max = dist_bias != nullptr && dist_max >= 0 ? dist_max : 0;
#define PRISM_MA_LAUNCH(DVP)                                                                                        \
    do {                                                                                                            \
        if (v_in_k) return few_rows ? launch_masked<DVP, true, true>(a, S, max_q_len, stream)                       \
                                    : launch_masked<DVP, true, false>(a, S, max_q_len, stream);                     \
        return few_rows ? launch_masked<DVP, false, true>(a, S, max_q_len, stream)                                  \
                        : launch_masked<DVP, false, false>(a, S, max_q_len, stream);                                \
    } while (0)
    if (dv <= 32) PRISM_MA_LAUNCH(32);
    if (dv <= 64) PRISM_MA_LAUNCH(64);
    if (dv <= 128) PRISM_MA_LAUNCH(128);
    PRISM_MA_LAUNCH(256);
#undef PRISM_MA_LAUNCH
}
