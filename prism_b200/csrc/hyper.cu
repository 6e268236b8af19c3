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

template <typename T>
__global__ void hyper_norm_kernel(const float* x_in, long long in_ss, float* x_out, long long out_ss,
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
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[PRISM_MAX_STREAMS];
#pragma unroll
        for (int i = 0; i < PRISM_MAX_STREAMS; ++i)
            if (i < s) x[i] = xi[(size_t)i * in_ss + c];
        float acc = 0.f;
        if (delta != nullptr) {
            float y = 0.f;
            for (int k = 0; k < nsplit; ++k) {
                const size_t at = (size_t)k * delta_ss + (size_t)t * W + c;
                y += delta_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(delta)[at])
                                : reinterpret_cast<const float*>(delta)[at];
            }
#pragma unroll
            for (int j = 0; j < PRISM_MAX_STREAMS; ++j) {
                if (j >= s) break;
                float v = 0.f;
#pragma unroll
                for (int i = 0; i < PRISM_MAX_STREAMS; ++i)
                    if (i < s) v = fmaf(cm[i * s + j], x[i], v);
                v = fmaf(co[j], y, v);
                if (write) x_out[(size_t)j * out_ss + (size_t)t * W + c] = v;
                acc = fmaf(ci[j], v, acc);
            }
        } else {
#pragma unroll
            for (int j = 0; j < PRISM_MAX_STREAMS; ++j) {
                if (j >= s) break;
                if (write) x_out[(size_t)j * out_ss + (size_t)t * W + c] = x[j];
                acc = fmaf(ci[j], x[j], acc);
            }
        }
        u[c] = acc;
        sum += acc;
    }
    if (weight == nullptr || h == nullptr) return;
    float mean = 0.f;
    if (!rms) mean = block_sum(sum, red) / (float)W;
    float sq = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float d = u[c] - mean;
        sq += d * d;
    }
    const float inv = 1.f / sqrtf(block_sum(sq, red) / (float)W + eps);
    T* ho = h + (size_t)blockIdx.x * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        ho[c] = from_float<T>((u[c] - mean) * inv * load_param(weight, weight_bf16, c));
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
    const int threads = W >= 4096 ? 512 : (W >= 1024 ? 256 : 128);
    const int b = PRISM_DTYPE_BF16;
#define PRISM_HN(TT)                                                                                                   \
    do {                                                                                                               \
        auto kern = prism::hyper_norm_kernel<TT>;                                                                      \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        return (int)prism::launch_kernel(kern, dim3(n), dim3(threads), smem, stream, x_in, in_ss, x_out, out_ss, delta, \
                                         delta_dtype == b, nsplit, delta_ss, mix, mix_dtype == b, outw, outw_dtype == b, \
                                         inw, inw_dtype == b, s, weight, weight_dtype == b, eps, rms, (TT*)h, rows, W);  \
    } while (0)
    if (h_dtype == PRISM_DTYPE_BF16) PRISM_HN(__nv_bfloat16);
    PRISM_HN(float);
#undef PRISM_HN
}
