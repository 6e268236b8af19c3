// Hyper-connections: the residual stream is s copies x_1 .. x_s [s, T, W] float32 instead of one.  Around a
// sublayer with result y (float32; possibly a stack of split partial sums):
//     read-in   u = sum_i in[i] x_i                       (what the sublayer's norm sees)
//     update    x_j <- sum_i mix[i][j] x_i + out[j] y     (all streams at once from the old ones)
// One kernel does the update that the previous sublayer left open and the read-in and norm of the next one, so
// every stream is read and written once per sublayer:
//     x <- update(x, y_prev);  u = read-in(x);  h = norm(u) * weight
// norm: layer norm without bias, (u - mean) / sqrt(mean((u - mean)^2) + eps), or RMS norm, u / sqrt(mean(u^2) + eps).
// Every part is optional: no y (nothing left open), no mix / out (identity and ones: with s = 1 this is the plain
// residual sum), no in (ones: the sum of the streams, as before the model's last norm), no weight (no norm: the
// update alone), and the input may be one row set read s times (a stream stride of 0: the copies at the start).
// With `rows` only the listed tokens are normed and the streams are not written back (the last norm of a step
// needs the rows whose logits are wanted, and nothing reads the streams after it).
// One CTA per token; u lives in shared memory between the passes; all arithmetic is float32.
#include "common.cuh"

#define PRISM_MAX_STREAMS 8

namespace prism {

// V = 4: W, the stream and split strides are multiples of 4 and every pointer is 16-byte aligned, so a thread moves
// four neighbouring columns at a time (128-bit loads and stores); V = 1 takes everything else.
// SMAX: the most copies this instantiation takes (its loops over copies are unrolled that far).
template <typename T, int V, int SMAX>
__global__ void __launch_bounds__(V == 4 ? 256 : 512) hyper_norm_kernel(const float* x_in, long long in_ss, float* x_out, long long out_ss,
                                  const void* __restrict__ delta_in, int delta_bf16, int nsplit, long long delta_ss,
                                  const void* __restrict__ mix, int mix_bf16, const void* __restrict__ outw, int outw_bf16,
                                  const void* __restrict__ inw, int inw_bf16, int s, const void* __restrict__ weight,
                                  int weight_bf16, float eps, int rms, T* __restrict__ h, const int* __restrict__ rows,
                                  int W) {
    pdl_trigger();
    extern __shared__ float sm[];
    float* u = sm;                              // [W]
    float* red = sm + W;                        // [33]
    float* cm = red + 33;                       // mix [s][s]
    float* co = cm + PRISM_MAX_STREAMS * PRISM_MAX_STREAMS;     // out [s]
    float* ci = co + PRISM_MAX_STREAMS;                         // in [s]
    // the connection weights do not depend on the step: read them before the dependency wait
    for (int i = threadIdx.x; i < s * s; i += blockDim.x)
        cm[i] = mix != nullptr ? load_param(mix, mix_bf16, i) : (i / s == i % s ? 1.f : 0.f);
    for (int i = threadIdx.x; i < s; i += blockDim.x) {
        co[i] = outw != nullptr ? load_param(outw, outw_bf16, i) : 1.f;
        ci[i] = inw != nullptr ? load_param(inw, inw_bf16, i) : 1.f;
    }
    pdl_wait();
    const int t = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    const float* xi = pdl_fresh(x_in) + (size_t)t * W;
    const void* delta = pdl_fresh(delta_in);
    const bool write = x_out != nullptr && rows == nullptr && (delta != nullptr || x_out != x_in || in_ss == 0);
    __syncthreads();
    float sum = 0.f;
    for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
        float x[SMAX][V];
#pragma unroll
        for (int i = 0; i < SMAX; ++i)
            if (i < s) {
                if (V == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(xi + (size_t)i * in_ss + c);
                    x[i][0] = v.x; x[i][V > 1 ? 1 : 0] = v.y; x[i][V > 2 ? 2 : 0] = v.z; x[i][V > 3 ? 3 : 0] = v.w;
                } else {
                    x[i][0] = xi[(size_t)i * in_ss + c];
                }
            }
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
        if (delta != nullptr) {
            float y[V];
#pragma unroll
            for (int e = 0; e < V; ++e) y[e] = 0.f;
            for (int k = 0; k < nsplit; ++k) {
                const size_t at = (size_t)k * delta_ss + (size_t)t * W + c;
                if (V == 4 && !delta_bf16) {
                    const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(delta) + at);
                    y[0] += v.x; y[V > 1 ? 1 : 0] += v.y; y[V > 2 ? 2 : 0] += v.z; y[V > 3 ? 3 : 0] += v.w;
                } else {
#pragma unroll
                    for (int e = 0; e < V; ++e)
                        y[e] += delta_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(delta)[at + e])
                                           : reinterpret_cast<const float*>(delta)[at + e];
                }
            }
#pragma unroll
            for (int j = 0; j < SMAX; ++j) {
                if (j >= s) break;
                float v[V];
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float w = 0.f;
#pragma unroll
                    for (int i = 0; i < SMAX; ++i)
                        if (i < s) w = fmaf(cm[i * s + j], x[i][e], w);
                    v[e] = fmaf(co[j], y[e], w);
                    acc[e] = fmaf(ci[j], v[e], acc[e]);
                }
                if (write) {
                    float* dst = x_out + (size_t)j * out_ss + (size_t)t * W + c;
                    if (V == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[V > 1 ? 1 : 0], v[V > 2 ? 2 : 0], v[V > 3 ? 3 : 0]);
                    else dst[0] = v[0];
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < SMAX; ++j) {
                if (j >= s) break;
                if (write) {
                    float* dst = x_out + (size_t)j * out_ss + (size_t)t * W + c;
                    if (V == 4) *reinterpret_cast<float4*>(dst) = make_float4(x[j][0], x[j][V > 1 ? 1 : 0], x[j][V > 2 ? 2 : 0], x[j][V > 3 ? 3 : 0]);
                    else dst[0] = x[j][0];
                }
#pragma unroll
                for (int e = 0; e < V; ++e) acc[e] = fmaf(ci[j], x[j][e], acc[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
            u[c + e] = acc[e];
            sum += acc[e];
        }
    }
    if (weight == nullptr || h == nullptr) return;
    float mean = 0.f;
    if (!rms) mean = block_sum(sum, red) / (float)W;
    float sq = 0.f;
    // a thread reads back the columns it wrote itself: no barrier needed before this pass
    for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float d = u[c + e] - mean;
            sq += d * d;
        }
    }
    const float inv = 1.f / sqrtf(block_sum(sq, red) / (float)W + eps);
    T* ho = h + (size_t)blockIdx.x * W;
    for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
        float r[V];
#pragma unroll
        for (int e = 0; e < V; ++e) r[e] = (u[c + e] - mean) * inv * load_param(weight, weight_bf16, c + e);
        if (V == 4 && sizeof(T) == 2) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[V > 1 ? 1 : 0]), hi = __floats2bfloat162_rn(r[V > 2 ? 2 : 0], r[V > 3 ? 3 : 0]);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(ho + c) = pk;
        } else {
#pragma unroll
            for (int e = 0; e < V; ++e) ho[c + e] = from_float<T>(r[e]);
        }
    }
}

}  // namespace prism

// x_in [s, T, W] float32 with stream stride in_ss (0: one [T, W] read s times); x_out [s, T, W] (stream stride out_ss;
// may be x_in; null: not written); delta [nsplit, T, W] float32 or bf16 (null: no update); mix [s, s] (from, to), outw
// [s], inw [s] (each may be null); weight [W] (null: no norm, h unused); h [n, W] of h_dtype; rows [n] or null (n = T).
PRISM_EXPORT int prism_hyper_norm(const float* x_in, long long in_ss, float* x_out, long long out_ss, const void* delta,
                                  int delta_dtype, int nsplit, long long delta_ss, const void* mix, int mix_dtype,
                                  const void* outw, int outw_dtype, const void* inw, int inw_dtype, int s, const void* weight,
                                  int weight_dtype, float eps, int rms, void* h, int h_dtype, const int* rows, int n, int W,
                                  cudaStream_t stream) {
    if (n <= 0 || W <= 0) return 0;
    if (s < 1 || s > PRISM_MAX_STREAMS) return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)W + 33 + PRISM_MAX_STREAMS * (PRISM_MAX_STREAMS + 2)) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int b = PRISM_DTYPE_BF16;
    const bool vec = s <= 4 && W % 4 == 0 && in_ss % 4 == 0 && out_ss % 4 == 0 && delta_ss % 4 == 0 && !((uintptr_t)x_in & 15) &&
                     !((uintptr_t)x_out & 15) && !((uintptr_t)delta & 15) && !((uintptr_t)h & 7);
    const int per = vec ? 4 : 1;
    const int threads = !vec && W >= 4096 ? 512 : (W / per >= 256 ? 256 : 128);
#define PRISM_HN(TT, V, SM)                                                                                              \
    do {                                                                                                               \
        auto kern = prism::hyper_norm_kernel<TT, V, SM>;                                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        return (int)prism::launch_kernel(kern, dim3(n), dim3(threads), smem, stream, x_in, in_ss, x_out, out_ss, delta, \
                                         delta_dtype == b, nsplit, delta_ss, mix, mix_dtype == b, outw, outw_dtype == b, \
                                         inw, inw_dtype == b, s, weight, weight_dtype == b, eps, rms, (TT*)h, rows, W);  \
    } while (0)
    if (vec && s <= 2) {
        if (h_dtype == PRISM_DTYPE_BF16) PRISM_HN(__nv_bfloat16, 4, 2);
        PRISM_HN(float, 4, 2);
    }
    if (vec && s <= 4) {
        if (h_dtype == PRISM_DTYPE_BF16) PRISM_HN(__nv_bfloat16, 4, 4);
        PRISM_HN(float, 4, 4);
    }
    if (h_dtype == PRISM_DTYPE_BF16) PRISM_HN(__nv_bfloat16, 1, PRISM_MAX_STREAMS);
    PRISM_HN(float, 1, PRISM_MAX_STREAMS);
#undef PRISM_HN
}
