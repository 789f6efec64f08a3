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

// A gated feed-forward's activation with clamps, on a [rows, 2 * width] input whose rows hold the gate half, then the up half:
//     g = min(gate + bias_g, limit);  u = clamp(up + bias_u, -limit, limit);  out = g * sigmoid(alpha * g) * (u + 1)
// (bias [2 * width] float32 or null).  The sums and the activation are float32.
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, const float* __restrict__ bias, int width,
                                   size_t total, float limit, float alpha) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t r = i / width;
    const int c = (int)(i - r * width);
    float g = to_float(gate_up[r * 2 * width + c]), u = to_float(gate_up[r * 2 * width + width + c]);
    if (bias) { g += bias[c]; u += bias[width + c]; }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    out[i] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

HYMT2_API int hymt2_clamped_glu(void* out, const void* gate_up, int dtype, const float* bias, int rows, int width, float limit, float alpha,
                                cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && width > 0 && limit > 0.f, "clamped_glu: bad sizes rows=%d width=%d limit=%g", rows, width, (double)limit);
    const size_t total = (size_t)rows * width;
    HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(clamped_glu_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (T*)out,
                                              (const T*)gate_up, bias, width, total, limit, alpha));
    return hymt2_check_launch("clamped_glu");
}

// Rotary positions on rows of heads that lie side by side: y[t, :cols] = x[t, :cols] with the first rot_dims entries of each of
// the first `heads` heads (d entries each) turned by angle = position * inv_freq[i]: pairing 0 pairs entry i with i + rot_dims/2,
// pairing 1 entry 2i with 2i + 1; (a, b) -> (a cos - b sin, b cos + a sin).  Columns behind the heads are copied.  y may have
// another type than x (float32: what enters a float32 recurrence is then never rounded), and may be x itself.
template <typename TX, typename TY>
__global__ void __launch_bounds__(128)
rotate_heads_kernel(TY* __restrict__ y, long ldy, const TX* __restrict__ x, long ldx, const int* __restrict__ token_pos,
                    const float* __restrict__ inv_freq, int heads, int d, int rot_dims, int pairing, int cols) {
    extern __shared__ float rot_cs[];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, half = rot_dims / 2;
    const int pos = token_pos[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, c;
        sincosf((float)pos * inv_freq[i], &sn, &c);
        rot_cs[2 * i] = c;
        rot_cs[2 * i + 1] = sn;
    }
    __syncthreads();
    const TX* src = x + (size_t)t * ldx;
    TY* dst = y + (size_t)t * ldy;
    const int per = half + (d - rot_dims);
    // (the blocks of a token share its heads and its copied columns among themselves)
    const int h_lo = (int)((long)heads * blockIdx.y / gridDim.y), h_hi = (int)((long)heads * (blockIdx.y + 1) / gridDim.y);
    for (int item = threadIdx.x; item < (h_hi - h_lo) * per; item += blockDim.x) {
        const int h = h_lo + item / per, i = item % per;
        const TX* s = src + (size_t)h * d;
        TY* o = dst + (size_t)h * d;
        if (i < half) {
            const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
            const float a = to_float(s[ia]), b = to_float(s[ib]);
            o[ia] = from_float<TY>(a * rot_cs[2 * i] - b * rot_cs[2 * i + 1]);
            o[ib] = from_float<TY>(b * rot_cs[2 * i] + a * rot_cs[2 * i + 1]);
        } else {
            const int e = rot_dims + (i - half);
            o[e] = from_float<TY>(to_float(s[e]));
        }
    }
    if ((const void*)src != (const void*)dst || sizeof(TX) != sizeof(TY))
        for (int c = heads * d + blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += blockDim.x * gridDim.y) dst[c] = from_float<TY>(to_float(src[c]));
}

HYMT2_API int hymt2_rotate_heads(void* y, int y_dtype, long ldy, const void* x, int x_dtype, long ldx, const int* token_pos,
                                 const float* inv_freq, int tokens, int heads, int d, int rot_dims, int pairing, int cols,
                                 cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && heads >= 0 && d > 0 && cols >= heads * d, "rotate_heads: bad sizes");
    HYMT2_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= d && (rot_dims == 0 || inv_freq != nullptr),
                  "rotate_heads: %d rotated entries of %d", rot_dims, d);
    const size_t smem = sizeof(float) * (size_t)(rot_dims + 2);
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(y_dtype, TY,
        (launch_pdl(rotate_heads_kernel<TX, TY>, dim3(tokens, tokens >= 512 ? 1 : (cols >= 2048 ? 8 : (cols >= 512 ? 2 : 1))), dim3(128), smem, stream, (TY*)y, ldy, (const TX*)x, ldx, token_pos, inv_freq,
                    heads, d, rot_dims, pairing, cols))));
    return hymt2_check_launch("rotate_heads");
}
