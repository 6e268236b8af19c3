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
// Further: the gated hidden layer out[t][i] = act(gu[t][i]) * gu[t][I + i] of a feed-forward whose gate and up
// projections are one product; out[t][c] = act(z[t][c]) * table[ids[t]][off + c], a gate on a slice of a row
// gathered per token; and the soft cap x <- cap tanh(x / cap) of float32 rows in place.
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

template <typename T, int ACT>
__global__ void glu_kernel(const T* __restrict__ gu_in, long long gs, T* __restrict__ out, long long os, int I, int vec) {
    pdl_trigger();
    pdl_wait();
    const T* gu = pdl_fresh(gu_in) + (size_t)blockIdx.y * gs;
    T* o = out + (size_t)blockIdx.y * os;
    if (vec) {                 // eight neighbouring columns a thread
        const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
        if (c >= I) return;
        float g[8], u[8];
        load8(gu + c, g);
        load8(gu + I + c, u);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = activate<ACT>(g[k]) * u[k];
        store8(o + c, g);
        return;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I; i += gridDim.x * blockDim.x)
        o[i] = from_float<T>(activate<ACT>(to_float(gu[i])) * to_float(gu[I + i]));
}

template <typename T, typename W, int ACT>
__global__ void gather_gate_kernel(const float* __restrict__ z_in, long long zs, const int* __restrict__ ids,
                                   const W* __restrict__ table, long long ts, int off, int V, T* __restrict__ out,
                                   long long os, int cols, int* err) {
    pdl_trigger();
    pdl_wait();
    const float* z = pdl_fresh(z_in) + (size_t)blockIdx.x * zs;
    const int id = pdl_fresh(ids)[blockIdx.x];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) report_error(err, PRISM_ERR_TOKEN_RANGE);
    T* o = out + (size_t)blockIdx.x * os;
    for (int c = threadIdx.x; c < cols; c += blockDim.x)
        o[c] = from_float<T>(ok ? activate<ACT>(z[c]) * to_float(table[(size_t)id * ts + off + c]) : 0.f);
}

__global__ void softcap_kernel(float* __restrict__ x_in, size_t n, float cap) {
    pdl_trigger();
    pdl_wait();
    float* x = pdl_fresh(x_in);
    const float inv = 1.f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
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

// gu [rows, 2 I] of `dtype` (gate columns first, row stride gu_stride) -> out [rows, I] = act(gate) * up.
// act: PRISM_ACT_SILU or PRISM_ACT_GELU_TANH.
PRISM_EXPORT int prism_glu(const void* gu, long long gu_stride, void* out, long long out_stride, int dtype, int rows, int I,
                           int act, cudaStream_t stream) {
    if (rows <= 0 || I <= 0) return 0;
    if (rows > 65535 || (act != PRISM_ACT_SILU && act != PRISM_ACT_GELU_TANH)) return (int)cudaErrorInvalidValue;
    const int esz = dtype == PRISM_DTYPE_BF16 ? 2 : 4;
    const bool vec = I % 8 == 0 && gu_stride % 8 == 0 && out_stride % 8 == 0 && (uintptr_t)gu % (8 * esz) == 0 &&
                     (uintptr_t)out % (8 * esz) == 0;
    dim3 grid(((vec ? I / 8 : I) + 255) / 256, rows);
#define PRISM_GLU(TT, A)                                                                                          \
    return (int)prism::launch_kernel(prism::glu_kernel<TT, A>, grid, dim3(256), 0, stream, (const TT*)gu, gu_stride, \
                                     (TT*)out, out_stride, I, vec ? 1 : 0)
    if (dtype == PRISM_DTYPE_BF16) {
        if (act == PRISM_ACT_SILU) PRISM_GLU(__nv_bfloat16, PRISM_ACT_SILU);
        PRISM_GLU(__nv_bfloat16, PRISM_ACT_GELU_TANH);
    }
    if (act == PRISM_ACT_SILU) PRISM_GLU(float, PRISM_ACT_SILU);
    PRISM_GLU(float, PRISM_ACT_GELU_TANH);
#undef PRISM_GLU
}

// z [rows, cols] float32; table [V, *] of table_dtype with row stride table_stride; out [rows, cols] of out_dtype:
// out[t][c] = act(z[t][c]) * table[ids[t]][off + c].  act: PRISM_ACT_GELU_TANH or PRISM_ACT_SILU.
PRISM_EXPORT int prism_gather_gate(const float* z, long long z_stride, const int* ids, const void* table, int table_dtype,
                                   long long table_stride, int off, int V, void* out, int out_dtype, long long out_stride,
                                   int rows, int cols, int act, int* err, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (act != PRISM_ACT_SILU && act != PRISM_ACT_GELU_TANH) return (int)cudaErrorInvalidValue;
    const int threads = cols >= 256 ? 256 : (cols >= 64 ? 64 : 32);
#define PRISM_GG(TT, WW, A)                                                                                          \
    return (int)prism::launch_kernel(prism::gather_gate_kernel<TT, WW, A>, dim3(rows), dim3(threads), 0, stream, z,   \
                                     z_stride, ids, (const WW*)table, table_stride, off, V, (TT*)out, out_stride, cols, err)
#define PRISM_GG_A(TT, WW)                                              \
    do {                                                                \
        if (act == PRISM_ACT_SILU) PRISM_GG(TT, WW, PRISM_ACT_SILU);    \
        PRISM_GG(TT, WW, PRISM_ACT_GELU_TANH);                          \
    } while (0)
    if (out_dtype == PRISM_DTYPE_BF16) {
        if (table_dtype == PRISM_DTYPE_BF16) PRISM_GG_A(__nv_bfloat16, __nv_bfloat16);
        PRISM_GG_A(__nv_bfloat16, float);
    }
    if (table_dtype == PRISM_DTYPE_BF16) PRISM_GG_A(float, __nv_bfloat16);
    PRISM_GG_A(float, float);
#undef PRISM_GG_A
#undef PRISM_GG
}

// x [n] float32 in place: x <- cap tanh(x / cap).
PRISM_EXPORT int prism_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    const long long blocks = (n + 255) / 256;
    return (int)prism::launch_kernel(prism::softcap_kernel, dim3((unsigned)(blocks < 148 * 8 ? blocks : 148 * 8)), dim3(256), 0,
                                     stream, x, (size_t)n, cap);
}
