// Paged causal grouped-query attention, shape-generic version: any head size
// up to 256, any page size, any number of heads and groups, float32 or bf16
// storage, optional sliding window.  It is the attention of the float32 path
// and the fallback of the bf16 path for shapes the tensor-core kernels refuse.
//
// For query token t of request seg at absolute position p, head h:
//     s_j = (q . k_j) * scale          for keys  max(0, p - window + 1) <= j <= p
//     o   = softmax(s) @ v             q-head h reads kv-head h / (nh / nkv)
// i.e. flash_attn_with_kvcache(causal=True) over the request's pages
// (andre-fu/prism engine/executor.py:119-120), with scores, running max and
// sum and the output accumulation in float32.  Keys are visited in blocks of
// 32 starting at the window's first key, so the order of additions for a
// position depends only on that position, not on how the request was cut
// into steps or on what else is in the batch.
//
// One warp per (token, head): each lane scores one key of the block, the
// block's probabilities are exchanged by shuffles, and each lane accumulates
// the output dims lane, lane+32, ...
#include "common.cuh"

namespace prism {

template <typename T> struct VecLoad;
template <> struct VecLoad<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ float dot(const float* __restrict__ a, const float* __restrict__ q) {
        const float4 v = *reinterpret_cast<const float4*>(a);
        return v.x * q[0] + v.y * q[1] + v.z * q[2] + v.w * q[3];
    }
};
template <> struct VecLoad<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ float dot(const __nv_bfloat16* __restrict__ a, const float* __restrict__ q) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            s += f.x * q[2 * i] + f.y * q[2 * i + 1];
        }
        return s;
    }
};

// Which keys the token at position p sees.  All three are causal (keys <= p):
//   MASK_CAUSAL  every key from 0;
//   MASK_WINDOW  the last `size` keys, p - size < key;
//   MASK_CHUNK   the keys of p's own block of `size` positions, blocks counted from position 0.
__host__ __device__ __forceinline__ int mask_first_key(int kind, int size, int pos) {
    if (kind == PRISM_MASK_WINDOW && size > 0) return pos - size + 1 > 0 ? pos - size + 1 : 0;
    if (kind == PRISM_MASK_CHUNK && size > 0) return pos / size * size;
    return 0;
}

// MAXD: output dims per lane, value size <= 32 * MAXD.  Keys of `dk` and values of `dv` entries per head may
// differ in size and live in planes with strides of their own (elements between tokens' rows and between
// heads), so that the values may also be a slice of the key rows.  `sink` (per query head, or null): one more
// term exp(sink_h) in the softmax's denominator, with no value; it is not multiplied by `scale`.
// `dist_bias` (float32 [nh, dist_max + 1], or null): a bias by distance, added to the scaled score of the key
// n = pos - j positions back: dist_bias[h][min(n, dist_max)] (distances beyond the table's end share its last entry).
template <typename T, int MAXD>
__global__ void attn_generic_kernel(const T* __restrict__ q, int q_stride, int q_head_stride, T* __restrict__ out,
                                    int out_stride, const T* __restrict__ kc, long long k_row_stride, int k_head_stride,
                                    const T* __restrict__ vc, long long v_row_stride, int v_head_stride,
                                    const int* __restrict__ block_table,
                                    int bt_width, const int* __restrict__ positions,
                                    const int* __restrict__ tok_seg, int Ttot, int nh, int nkv,
                                    int dk, int dv, int page_size, int num_pages, int mask_kind, int mask_size,
                                    int mask_keep, float scale, const void* __restrict__ sink, int sink_bf16, int* err,
                                    const float* __restrict__ dist_bias, int dist_max) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (w >= (long long)Ttot * nh) return;
    const int t = (int)(w / nh), h = (int)(w % nh);
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* bt = block_table + (size_t)tok_seg[t] * bt_width;
    const int lo = mask_first_key(mask_kind, mask_size, pos);
    // the first `mask_keep` positions stay visible behind a window: they are visited first, in blocks of 32 from
    // key 0, then the window's keys from its first key - an order that depends on the position only
    const int keep = mask_keep < lo ? mask_keep : lo;

    float* qs = smem + warp * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_float(q[(size_t)t * q_stride + (size_t)h * q_head_stride + d]);
    __syncwarp();

    float acc[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    constexpr int VN = VecLoad<T>::N;
    const bool vec_ok = dk % VN == 0 && k_row_stride % VN == 0 && k_head_stride % VN == 0 &&
                        (reinterpret_cast<uintptr_t>(kc) % (VN * sizeof(T))) == 0;

    for (int kb = keep > 0 ? 0 : lo; kb <= pos; kb = (kb < lo && kb + 32 >= keep) ? lo : kb + 32) {
        const int j = kb + lane;
        const int last = kb < lo ? keep - 1 : pos;     // the last key of the run this block lies in
        bool valid = j <= last;
        int rowidx = -1;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                report_error(err, PRISM_ERR_PAGE_RANGE);
                valid = false;
            } else {
                rowidx = page * page_size + j % page_size;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = kc + (size_t)rowidx * k_row_stride + (size_t)kvh * k_head_stride;
            float dot = 0.f;
            if (vec_ok) {
                for (int d = 0; d < dk; d += VN) dot += VecLoad<T>::dot(kr + d, qs + d);
            } else {
                for (int d = 0; d < dk; ++d) dot += qs[d] * to_float(kr[d]);
            }
            s = dot * scale;
            if (dist_bias != nullptr) s += dist_bias[(size_t)h * (dist_max + 1) + min(pos - j, dist_max)];
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;            // only after a page error
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAXD; ++i) acc[i] *= corr;
        const int cnt = min(32, last - kb + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int rj = __shfl_sync(0xffffffffu, rowidx, jj);
            if (rj < 0) continue;
            const T* vr = vc + (size_t)rj * v_row_stride + (size_t)kvh * v_head_stride;
#pragma unroll
            for (int i = 0; i < MAXD; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] += pj * to_float(vr[d]);
            }
        }
        m = m_new;
    }
    if (sink != nullptr) {
        const float sk = load_param(sink, sink_bf16, h);
        const float m_all = fmaxf(m, sk);
        const float corr = expf(m - m_all);          // 0 when no key was seen
        l = l * corr + expf(sk - m_all);
#pragma unroll
        for (int i = 0; i < MAXD; ++i) acc[i] *= corr;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAXD; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) out[(size_t)t * out_stride + (size_t)h * dv + d] = from_float<T>(acc[i] * inv);
    }
}

template <typename T, int MAXD>
static int launch_generic(const void* q, int q_stride, int q_head_stride, void* out, int out_stride, const void* kc,
                          long long k_row_stride, int k_head_stride, const void* vc, long long v_row_stride,
                          int v_head_stride, const int* block_table, int bt_width, const int* positions,
                          const int* tok_seg, int T_, int nh, int nkv, int dk, int dv, int page_size, int num_pages,
                          int mask_kind, int mask_size, int mask_keep, float scale, const void* sink, int sink_bf16,
                          int* err, const float* dist_bias, int dist_max, cudaStream_t stream) {
    const int warps = 4;
    const long long total = (long long)T_ * nh;
    const int blocks = (int)((total + warps - 1) / warps);
    const size_t smem = (size_t)warps * dk * sizeof(float);
    auto kern = attn_generic_kernel<T, MAXD>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<blocks, warps * 32, smem, stream>>>(
        (const T*)q, q_stride, q_head_stride, (T*)out, out_stride, (const T*)kc, k_row_stride, k_head_stride,
        (const T*)vc, v_row_stride, v_head_stride, block_table, bt_width, positions, tok_seg, T_, nh, nkv, dk, dv,
        page_size, num_pages, mask_kind, mask_size, mask_keep, scale, sink, sink_bf16, err, dist_bias, dist_max);
    return (int)cudaPeekAtLastError();
}

}  // namespace prism

// Keys of dk and values of dv entries, each plane with its own strides (in elements: between the rows of
// consecutive cache slots, and between kv heads); mask_kind PRISM_MASK_*; mask_keep: under PRISM_MASK_WINDOW
// the first mask_keep positions stay visible to every later query; sink: per-head float32 or bf16
// (sink_dtype) or null; dist_bias: float32 [nh, dist_max + 1] or null.  Returns cudaErrorInvalidValue for dv > 1024 or dk > 12288 / warps.
PRISM_EXPORT int prism_attention_masked_generic(const void* q, int q_stride, int q_head_stride, void* out,
                                                int out_stride, const void* kc, long long k_row_stride,
                                                int k_head_stride, const void* vc, long long v_row_stride,
                                                int v_head_stride, int dtype, const int* block_table, int bt_width,
                                                const int* positions, const int* tok_seg, int T, int nh, int nkv,
                                                int dk, int dv, int page_size, int num_pages, int mask_kind,
                                                int mask_size, int mask_keep, float scale, const void* sink,
                                                int sink_dtype, int* err, const float* dist_bias, int dist_max,
                                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dist_bias != nullptr && dist_max < 0) return (int)cudaErrorInvalidValue;
    if (mask_keep < 0 || (mask_keep > 0 && mask_kind != PRISM_MASK_WINDOW)) return (int)cudaErrorInvalidValue;
    if (dv > 1024 || dv <= 0 || dk <= 0 || dk > 8192 || nkv <= 0 || nh % nkv != 0) return (int)cudaErrorInvalidValue;
    const int sb = sink_dtype == PRISM_DTYPE_BF16;
#define PRISM_GENERIC(TT, MD)                                                                                       \
    return prism::launch_generic<TT, MD>(q, q_stride, q_head_stride, out, out_stride, kc, k_row_stride,             \
                                         k_head_stride, vc, v_row_stride, v_head_stride, block_table, bt_width,     \
                                         positions, tok_seg, T, nh, nkv, dk, dv, page_size, num_pages, mask_kind,   \
                                         mask_size, mask_keep, scale, sink, sb, err, dist_bias, dist_max, stream)
    if (dtype == PRISM_DTYPE_BF16) {
        if (dv <= 256) PRISM_GENERIC(__nv_bfloat16, 8);
        if (dv <= 512) PRISM_GENERIC(__nv_bfloat16, 16);
        PRISM_GENERIC(__nv_bfloat16, 32);
    }
    if (dv <= 256) PRISM_GENERIC(float, 8);
    if (dv <= 512) PRISM_GENERIC(float, 16);
    PRISM_GENERIC(float, 32);
#undef PRISM_GENERIC
}

// Keys and values of one size hd in planes [slots, nkv, hd]; window <= 0: all keys.  Returns
// cudaErrorInvalidValue for head_dim > 256.
PRISM_EXPORT int prism_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                         const void* kc, const void* vc, int dtype,
                                         const int* block_table, int bt_width,
                                         const int* positions, const int* tok_seg, int T, int nh,
                                         int nkv, int hd, int page_size, int num_pages, int window,
                                         float scale, int* err, cudaStream_t stream) {
    if (hd > 256) return (int)cudaErrorInvalidValue;
    return prism_attention_masked_generic(q, q_stride, hd, out, out_stride, kc, (long long)nkv * hd, hd, vc,
                                          (long long)nkv * hd, hd, dtype, block_table, bt_width, positions, tok_seg,
                                          T, nh, nkv, hd, hd, page_size, num_pages,
                                          window > 0 ? PRISM_MASK_WINDOW : PRISM_MASK_CAUSAL, window, 0, scale, nullptr, 0,
                                          err, nullptr, 0, stream);
}
