// Query/key norm, rotation and cache store for attention layers that norm each head of q and k before they
// rotate it.  From the float32 result of the input projection, per token:
//   q_h <- rotate(q_h / sqrt(mean(q_h^2) + eps) * wq)      into q_out [T, nh, dk] (compute dtype)
//   k_g <- rotate(k_g / sqrt(mean(k_g^2) + eps) * wk)      into the key plane, at the token's slot
//   v_g                                                    into the value plane, at the token's slot
// wq, wk: one weight vector of dk entries each, shared by the heads (null: no norm).  With `whole` the norm runs
// over the whole projection instead, all heads of q (of k) at once, q <- q / sqrt(mean over nh dk (q^2) + eps) * wq
// with wq of nh dk entries (wk: nkv dk).  The rotation turns the
// first `rot` entries of a head, entry 2i paired with entry 2i + 1 (interleaved pairs) or, with `halves`, entry i
// with entry i + rot / 2: the pair (a, b) at
// position p becomes (a cos t - b sin t, b cos t + a sin t), t = p * freq[i]; `freq` is a float32 table
// of rot / 2 entries (any frequency scaling is in the table), the angle and sincosf are float32.  The slot of
// position p of request seg is block_table[seg][p / page_size] * page_size + p % page_size.
// One warp per (token, head); one more warp per token copies the values.
#include "common.cuh"

namespace prism {

template <typename T>
__global__ void qk_norm_rope_store_kernel(const float* __restrict__ q_in, const float* __restrict__ k_in,
                                          const float* __restrict__ v_in, long long ps, const void* __restrict__ wq,
                                          int wq_bf16, const void* __restrict__ wk, int wk_bf16, float eps,
                                          const float* __restrict__ freq, int rot, T* __restrict__ q_out,
                                          T* __restrict__ k_plane, T* __restrict__ v_plane,
                                          const int* __restrict__ block_table, int bt_width,
                                          const int* __restrict__ positions, const int* __restrict__ tok_seg, int nh, int nkv,
                                          int dk, int dv, int page_size, int num_pages, int max_pos, int* err, int whole,
                                          int halves) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float* q = pdl_fresh(q_in) + (size_t)t * ps;
    const float* k = pdl_fresh(k_in) + (size_t)t * ps;
    const float* v = pdl_fresh(v_in) + (size_t)t * ps;
    const int pos = positions[t];
    float inv_q = 1.f, inv_k = 1.f;           // whole: every CTA of the token forms both sums itself
    if (whole && (wq != nullptr || wk != nullptr)) {
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < nh * dk; c += blockDim.x) sq += q[c] * q[c];
        if (k_plane != nullptr)
            for (int c = threadIdx.x; c < nkv * dk; c += blockDim.x) sk += k[c] * k[c];
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        inv_q = 1.f / sqrtf(sq / (float)(nh * dk) + eps);
        inv_k = 1.f / sqrtf(sk / (float)(nkv * dk) + eps);
    }
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_POSITION_RANGE);
        return;
    }
    // a layer without planes of its own stores nothing and looks up no page
    const int page = k_plane != nullptr ? block_table[(size_t)tok_seg[t] * bt_width + pos / page_size] : 0;
    const bool page_ok = page >= 0 && page < num_pages;
    if (!page_ok && threadIdx.x == 0) report_error(err, PRISM_ERR_PAGE_RANGE);
    const size_t slot = page_ok ? (size_t)page * page_size + pos % page_size : 0;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);      // q heads, k heads, then the values
    if (unit == nh + nkv && page_ok && v_plane != nullptr)
        for (int c = lane; c < nkv * dv; c += 32) v_plane[slot * nkv * dv + c] = from_float<T>(v[c]);
    const int half = rot >> 1;
    for (int hh = unit; hh < nh + nkv; hh += nh + nkv) {
        const bool is_q = hh < nh;
        if (!is_q && k_plane == nullptr) continue;          // a layer that reads another layer's keys and values
        const float* row = is_q ? q + (size_t)hh * dk : k + (size_t)(hh - nh) * dk;
        const void* w = is_q ? wq : wk;
        const int wb = is_q ? wq_bf16 : wk_bf16;
        const size_t w0 = whole ? (size_t)(is_q ? hh : hh - nh) * dk : 0;      // the head's first weight
        float inv = is_q ? inv_q : inv_k;
        if (w != nullptr && !whole) {
            float ss = 0.f;
            for (int d = lane; d < dk; d += 32) ss += row[d] * row[d];
            ss = warp_sum(ss);
            inv = 1.f / sqrtf(ss / (float)dk + eps);
        }
        if (!is_q && !page_ok) continue;
        T* dst = is_q ? q_out + ((size_t)t * nh + hh) * dk : k_plane + (slot * nkv + (hh - nh)) * dk;
        for (int d = lane; d < dk; d += 32) {
            float a = row[d] * inv * (w != nullptr ? load_param(w, wb, w0 + d) : 1.f);
            if (d < rot) {
                const int e = halves ? (d < half ? d + half : d - half) : d ^ 1;
                const bool second = halves ? d >= half : (d & 1);
                const float b = row[e] * inv * (w != nullptr ? load_param(w, wb, w0 + e) : 1.f);
                float sn, cs;
                sincosf((float)pos * freq[halves ? (second ? e : d) : d >> 1], &sn, &cs);
                a = second ? a * cs + b * sn : a * cs - b * sn;
            }
            dst[d] = from_float<T>(a);
        }
    }
}

}  // namespace prism

// q, k, v: float32 rows with one row stride `ps` (column blocks of one product); planes [slots, nkv, dk] and
// [slots, nkv, dv] of `dtype` (both null: only q is made), q_out [T, nh, dk] of `dtype`; rot even, <= dk.
PRISM_EXPORT int prism_qk_norm_rope_store(const float* q, const float* k, const float* v, long long ps, const void* wq,
                                          int wq_dtype, const void* wk, int wk_dtype, float eps, const float* freq, int rot,
                                          void* q_out, void* k_plane, void* v_plane, int dtype, const int* block_table,
                                          int bt_width, const int* positions, const int* tok_seg, int T, int nh, int nkv, int dk,
                                          int dv, int page_size, int num_pages, int max_pos, int* err, int whole, int halves,
                                          cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > dk || rot % 2 || (rot > 0 && freq == nullptr) || nh < 1 || nkv < 1 || dk < 1 || dv < 1)
        return (int)cudaErrorInvalidValue;
    const int units = nh + nkv + 1;
    const int threads = units >= 4 ? 128 : 32 * units;
    const dim3 grid(T, (units + threads / 32 - 1) / (threads / 32));
    if (T > 65535 * 32) return (int)cudaErrorInvalidValue;
    const int qb = wq_dtype == PRISM_DTYPE_BF16, kb = wk_dtype == PRISM_DTYPE_BF16;
    if (dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::qk_norm_rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, q, k,
                                         v, ps, wq, qb, wk, kb, eps, freq, rot, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_plane,
                                         (__nv_bfloat16*)v_plane, block_table, bt_width, positions, tok_seg, nh, nkv, dk, dv,
                                         page_size, num_pages, max_pos, err, whole, halves);
    return (int)prism::launch_kernel(prism::qk_norm_rope_store_kernel<float>, grid, dim3(threads), 0, stream, q, k, v, ps, wq,
                                     qb, wk, kb, eps, freq, rot, (float*)q_out, (float*)k_plane, (float*)v_plane, block_table,
                                     bt_width, positions, tok_seg, nh, nkv, dk, dv, page_size, num_pages, max_pos, err, whole, halves);
}
