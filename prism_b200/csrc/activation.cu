// Elementwise activations of a feed-forward's hidden layer: out[i] = act(x[i]), float32 arithmetic, one
// rounding at the store.
//   PRISM_ACT_RELU2      max(z, 0)^2
//   PRISM_ACT_GELU_TANH  0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   PRISM_ACT_SILU       z / (1 + exp(-z))
//   PRISM_ACT_RELU       max(z, 0)
//   PRISM_ACT_TANH       tanh(z)
//   PRISM_ACT_SIGMOID    1 / (1 + exp(-z))
// and the gated product out[i] = x[i] * act(g[i]) * c, with the gate g in float32 (a projection's float32
// result) whatever the dtype of x and out; one gate entry may cover `group` neighbouring columns (a gate per head).
// Input and output rows may have strides of their own (the output may be a column block of a wider buffer).
#include "common.cuh"
#include "vec.cuh"

#define PRISM_ACT_RELU2 0
#define PRISM_ACT_GELU_TANH 1
#define PRISM_ACT_SILU 2
#define PRISM_ACT_RELU 3
#define PRISM_ACT_TANH 4
#define PRISM_ACT_SIGMOID 5

namespace prism {

template <int ACT> __device__ __forceinline__ float activate(float z) {
    if (ACT == PRISM_ACT_RELU2) {
        const float r = fmaxf(z, 0.f);
        return r * r;
    }
    if (ACT == PRISM_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    if (ACT == PRISM_ACT_SILU) return z / (1.f + expf(-z));
    if (ACT == PRISM_ACT_TANH) return tanhf(z);
    if (ACT == PRISM_ACT_SIGMOID) return 1.f / (1.f + expf(-z));
    return fmaxf(z, 0.f);
}

template <typename T, int ACT>
__global__ void activation_kernel(const T* __restrict__ x_in, long long x_stride, T* __restrict__ out,
                                  long long out_stride, int rows, int cols, int vec) {
    pdl_trigger();
    pdl_wait();
    const T* x = pdl_fresh(x_in);
    const int r = blockIdx.y;
    if (vec) {
        const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
        if (c >= cols) return;
        float v[8];
        load8(x + (size_t)r * x_stride + c, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = activate<ACT>(v[k]);
        store8(out + (size_t)r * out_stride + c, v);
        return;
    }
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x)
        out[(size_t)r * out_stride + c] = from_float<T>(activate<ACT>(to_float(x[(size_t)r * x_stride + c])));
}

template <typename T>
static int launch_activation(const void* x, long long xs, void* out, long long os, int rows, int cols, int act,
                             cudaStream_t stream) {
    const bool vec = cols % 8 == 0 && xs % 8 == 0 && os % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (sizeof(T) == 2 || ((uintptr_t)x % 32 == 0 && (uintptr_t)out % 32 == 0));
    const int per = vec ? cols / 8 : cols;
    dim3 grid((per + 255) / 256, rows);
#define PRISM_ACT_LAUNCH(A)                                                                                    \
    return (int)launch_kernel(activation_kernel<T, A>, grid, dim3(256), 0, stream, (const T*)x, xs, (T*)out, os, rows, \
                              cols, vec ? 1 : 0)
    switch (act) {
        case PRISM_ACT_RELU2: PRISM_ACT_LAUNCH(PRISM_ACT_RELU2);
        case PRISM_ACT_GELU_TANH: PRISM_ACT_LAUNCH(PRISM_ACT_GELU_TANH);
        case PRISM_ACT_SILU: PRISM_ACT_LAUNCH(PRISM_ACT_SILU);
        case PRISM_ACT_RELU: PRISM_ACT_LAUNCH(PRISM_ACT_RELU);
        case PRISM_ACT_TANH: PRISM_ACT_LAUNCH(PRISM_ACT_TANH);
        case PRISM_ACT_SIGMOID: PRISM_ACT_LAUNCH(PRISM_ACT_SIGMOID);
    }
#undef PRISM_ACT_LAUNCH
    return (int)cudaErrorInvalidValue;
}

template <typename T, int ACT>
__global__ void gated_product_kernel(const T* __restrict__ x_in, long long x_stride, const float* __restrict__ g_in,
                                     long long g_stride, T* __restrict__ out, long long out_stride, int cols, float c,
                                     int group) {
    pdl_trigger();
    pdl_wait();
    const T* x = pdl_fresh(x_in) + (size_t)blockIdx.y * x_stride;
    const float* g = pdl_fresh(g_in) + (size_t)blockIdx.y * g_stride;
    T* o = out + (size_t)blockIdx.y * out_stride;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < cols; i += gridDim.x * blockDim.x)
        o[i] = from_float<T>(to_float(x[i]) * activate<ACT>(g[i / group]) * c);
}

}  // namespace prism

// out = x * act(gate) * c; x and out [rows, cols] of `dtype`, gate [rows, cols / group] float32, each with a row stride
// of its own.
// act: PRISM_ACT_SIGMOID or PRISM_ACT_SILU.
PRISM_EXPORT int prism_gated_product(const void* x, long long x_stride, const float* gate, long long gate_stride, void* out,
                                     long long out_stride, int dtype, int rows, int cols, int act, float c, int group,
                                     cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (group < 1 || rows > 65535 || (act != PRISM_ACT_SIGMOID && act != PRISM_ACT_SILU)) return (int)cudaErrorInvalidValue;
    dim3 grid((cols + 255) / 256, rows);
#define PRISM_GP(TT, A)                                                                                              \
    return (int)prism::launch_kernel(prism::gated_product_kernel<TT, A>, grid, dim3(256), 0, stream, (const TT*)x,    \
                                     x_stride, gate, gate_stride, (TT*)out, out_stride, cols, c, group)
    if (dtype == PRISM_DTYPE_BF16) {
        if (act == PRISM_ACT_SIGMOID) PRISM_GP(__nv_bfloat16, PRISM_ACT_SIGMOID);
        PRISM_GP(__nv_bfloat16, PRISM_ACT_SILU);
    }
    if (act == PRISM_ACT_SIGMOID) PRISM_GP(float, PRISM_ACT_SIGMOID);
    PRISM_GP(float, PRISM_ACT_SILU);
#undef PRISM_GP
}

PRISM_EXPORT int prism_activation(const void* x, long long x_stride, void* out, long long out_stride, int dtype,
                                  int rows, int cols, int act, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (rows > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == PRISM_DTYPE_BF16)
        return prism::launch_activation<__nv_bfloat16>(x, x_stride, out, out_stride, rows, cols, act, stream);
    return prism::launch_activation<float>(x, x_stride, out, out_stride, rows, cols, act, stream);
}
