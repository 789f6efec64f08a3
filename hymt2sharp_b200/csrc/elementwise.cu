// Small element-by-element steps between the products of a layer.  All arithmetic is float32; the rows may be
// views into wider buffers (a leading dimension comes with every matrix).
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_e(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// x[r, c] <- act(x[r, c] + bias[c]); the first `act_cols` columns get the tanh form of GELU, the others the bias alone.
// A thread takes V neighbouring columns (cols is a multiple of V).
template <typename T, int V>
__global__ void bias_act_kernel(T* __restrict__ x, const float* __restrict__ bias, int cols, long ld, int act_cols, size_t total) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (i >= total) return;
    const size_t r = i / cols;
    const int c = (int)(i - r * cols);
    T* px = x + r * ld + c;
    Pack<T, V> pk = load_pack<T, V>(px);
#pragma unroll
    for (int k = 0; k < V; k++) {
        float v = to_float(pk.v[k]) + (bias ? bias[c + k] : 0.f);
        if (c + k < act_cols) v = gelu_tanh_f(v);
        pk.v[k] = from_float<T>(v);
    }
    store_pack<T, V>(px, pk);
}

// xIELU with its two numbers (p, q) read from the device: for z > 0  softplus(p) z^2 + z / 2;
// for z <= 0  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
template <typename T, int V>
__global__ void xielu_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ pq, size_t total) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (i >= total) return;
    const float ap = softplus_e(pq[0]), an = 0.5f + softplus_e(pq[1]);
    Pack<T, V> pk = load_pack<T, V>(x + i);
#pragma unroll
    for (int k = 0; k < V; k++) {
        const float z = to_float(pk.v[k]);
        pk.v[k] = from_float<T>(z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z));
    }
    store_pack<T, V>(out + i, pk);
}

// The square of relu: max(z, 0)^2.
template <typename T, int V>
__global__ void relu_squared_kernel(T* __restrict__ out, const T* __restrict__ x, size_t total) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (i >= total) return;
    Pack<T, V> pk = load_pack<T, V>(x + i);
#pragma unroll
    for (int k = 0; k < V; k++) {
        const float z = fmaxf(to_float(pk.v[k]), 0.f);
        pk.v[k] = from_float<T>(z * z);
    }
    store_pack<T, V>(out + i, pk);
}

// out = x rounded to out's type
template <typename TO, typename TI>
__global__ void convert_kernel(TO* __restrict__ out, const TI* __restrict__ x, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<TO>(to_float(x[i]));
}

// x[t, h, v] <- x[t, h, v] * sigmoid(g[t, per_head ? h : h * vdim + v])
template <typename T, int V>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const T* __restrict__ g, int heads, int vdim, long ldg, int per_head,
                                    size_t total) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;   // V neighbours of one head (vdim is a multiple of V)
    if (i >= total) return;
    const int width = heads * vdim;
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    Pack<T, V> pk = load_pack<T, V>(x + i);
    if (per_head) {
        const float s = 1.0f / (1.0f + expf(-to_float(g[t * ldg + c / vdim])));
#pragma unroll
        for (int k = 0; k < V; k++) pk.v[k] = from_float<T>(to_float(pk.v[k]) * s);
    } else {
#pragma unroll
        for (int k = 0; k < V; k++) pk.v[k] = from_float<T>(to_float(pk.v[k]) / (1.0f + expf(-to_float(g[t * ldg + c + k]))));
    }
    store_pack<T, V>(x + i, pk);
}

// x <- cap * tanh(x / cap)
__global__ void softcap_kernel(float* __restrict__ x, float cap, size_t total) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    x[i] = cap * tanhf(x[i] / cap);
}

inline unsigned blocks_for(size_t total) { return (unsigned)((total + 255) / 256); }

// out[r, c] = act(gu[r, c]) * gu[r, width + c] on rows that hold a gate half and an up half side by side; act: 0 silu,
// 1 the tanh form of GELU.  A thread takes V neighbouring columns.
template <typename T, int V>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ gu, int width, int kind, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (i >= total) return;
    const size_t r = i / width;
    const int c = (int)(i - r * width);
    const Pack<T, V> g = load_pack<T, V>(gu + r * 2 * width + c), u = load_pack<T, V>(gu + r * 2 * width + width + c);
    Pack<T, V> o;
#pragma unroll
    for (int k = 0; k < V; k++) {
        const float z = to_float(g.v[k]);
        const float a = kind == 0 ? z / (1.0f + expf(-z)) : gelu_tanh_f(z);
        o.v[k] = from_float<T>(a * to_float(u.v[k]));
    }
    store_pack<T, V>(out + i, o);
}

__global__ void tanh_kernel(float* __restrict__ x, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = tanhf(x[i]);
}

}  // namespace

HYMT2_API int hymt2_bias_act(void* x, int dtype, const float* bias, int rows, int cols, long ld, int act_cols, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && cols > 0 && ld >= cols && act_cols >= 0 && act_cols <= cols, "bias_act: bad sizes");
    const size_t total = (size_t)rows * cols;
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (cols % V == 0 && ld % V == 0 && (uintptr_t)x % 16 == 0)
            launch_pdl(bias_act_kernel<T, V>, dim3(blocks_for(total / V)), dim3(256), 0, stream, (T*)x, bias, cols, ld, act_cols, total);
        else
            launch_pdl(bias_act_kernel<T, 1>, dim3(blocks_for(total)), dim3(256), 0, stream, (T*)x, bias, cols, ld, act_cols, total);
    });
    return hymt2_check_launch("bias_act");
}

HYMT2_API int hymt2_xielu(void* out, const void* x, int dtype, const float* pq, long total, cudaStream_t stream) {
    if (total == 0) return HYMT2_OK;
    HYMT2_REQUIRE(total > 0 && pq != nullptr, "xielu: bad sizes");
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (total % V == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0)
            launch_pdl(xielu_kernel<T, V>, dim3(blocks_for((size_t)total / V)), dim3(256), 0, stream, (T*)out, (const T*)x, pq, (size_t)total);
        else
            launch_pdl(xielu_kernel<T, 1>, dim3(blocks_for((size_t)total)), dim3(256), 0, stream, (T*)out, (const T*)x, pq, (size_t)total);
    });
    return hymt2_check_launch("xielu");
}

HYMT2_API int hymt2_relu_squared(void* out, const void* x, int dtype, long total, cudaStream_t stream) {
    if (total == 0) return HYMT2_OK;
    HYMT2_REQUIRE(total > 0, "relu_squared: bad sizes");
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (total % V == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0)
            launch_pdl(relu_squared_kernel<T, V>, dim3(blocks_for((size_t)total / V)), dim3(256), 0, stream, (T*)out, (const T*)x, (size_t)total);
        else
            launch_pdl(relu_squared_kernel<T, 1>, dim3(blocks_for((size_t)total)), dim3(256), 0, stream, (T*)out, (const T*)x, (size_t)total);
    });
    return hymt2_check_launch("relu_squared");
}

HYMT2_API int hymt2_convert(void* out, int out_dtype, const void* x, int x_dtype, long total, cudaStream_t stream) {
    if (total == 0) return HYMT2_OK;
    HYMT2_REQUIRE(total > 0, "convert: bad sizes");
    HYMT2_DISPATCH_DTYPE(out_dtype, TO, HYMT2_DISPATCH_DTYPE(x_dtype, TI,
        (launch_pdl(convert_kernel<TO, TI>, dim3(blocks_for((size_t)total)), dim3(256), 0, stream, (TO*)out, (const TI*)x, (size_t)total))));
    return hymt2_check_launch("convert");
}

HYMT2_API int hymt2_sigmoid_gate(void* x, const void* g, int dtype, int rows, int heads, int vdim, long ldg, int per_head,
                                 cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && heads > 0 && vdim > 0, "sigmoid_gate: bad sizes");
    const size_t total = (size_t)rows * heads * vdim;
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (vdim % V == 0 && (uintptr_t)x % 16 == 0)
            launch_pdl(sigmoid_gate_kernel<T, V>, dim3(blocks_for(total / V)), dim3(256), 0, stream, (T*)x, (const T*)g, heads, vdim, ldg, per_head, total);
        else
            launch_pdl(sigmoid_gate_kernel<T, 1>, dim3(blocks_for(total)), dim3(256), 0, stream, (T*)x, (const T*)g, heads, vdim, ldg, per_head, total);
    });
    return hymt2_check_launch("sigmoid_gate");
}

HYMT2_API int hymt2_softcap(float* x, float cap, long total, cudaStream_t stream) {
    if (total == 0) return HYMT2_OK;
    HYMT2_REQUIRE(total > 0 && cap > 0.f, "softcap: bad arguments");
    launch_pdl(softcap_kernel, dim3(blocks_for((size_t)total)), dim3(256), 0, stream, x, cap, (size_t)total);
    return hymt2_check_launch("softcap");
}

HYMT2_API int hymt2_gated_act(void* out, const void* gate_up, int dtype, int rows, int width, int kind, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && width > 0 && (kind == 0 || kind == 1), "gated_act: bad arguments");
    const size_t total = (size_t)rows * width;
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (width % V == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0)
            launch_pdl(gated_act_kernel<T, V>, dim3(blocks_for(total / V)), dim3(256), 0, stream, (T*)out, (const T*)gate_up, width, kind, total);
        else
            launch_pdl(gated_act_kernel<T, 1>, dim3(blocks_for(total)), dim3(256), 0, stream, (T*)out, (const T*)gate_up, width, kind, total);
    });
    return hymt2_check_launch("gated_act");
}

HYMT2_API int hymt2_tanh(float* x, long total, cudaStream_t stream) {
    if (total == 0) return HYMT2_OK;
    HYMT2_REQUIRE(total > 0, "tanh: bad sizes");
    launch_pdl(tanh_kernel, dim3(blocks_for((size_t)total)), dim3(256), 0, stream, x, (size_t)total);
    return hymt2_check_launch("tanh");
}
