// Layer norm with a gain and no bias, row by row, all in float32:
//     y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * gain
// (the variance is the mean of the squared deviations, taken in a pass of its own after the mean), in the forms that a
// block with norms before AND after its sublayers needs: stored (optionally of gathered rows, optionally scaled), added
// into float32 rows, and "added, then the next norm of the new rows" in one launch.  And the sum of several branches, each
// divided by its own root mean square and multiplied by its own gain: out = sum_b scale_b * x_b / sqrt(mean(x_b^2) + eps) * gain_b.
// One block per row.  Rows of up to 8,192 entries stay in registers between the passes (eight entries a thread); wider rows are
// read from global memory in every pass (they stay in L1/L2 between them).
#include "common.cuh"

namespace {

template <typename TX>
__device__ __forceinline__ void row_moments(const TX* __restrict__ src, int dim, float* scratch, float& mean, float& var) {
    float s = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) s += to_float(src[i]);
    mean = block_sum(s, scratch) / (float)dim;
    float q = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = to_float(src[i]) - mean;
        q = fmaf(d, d, q);
    }
    var = block_sum(q, scratch) / (float)dim;
}

template <typename TX, typename TW, typename TY, bool ADD>
__global__ void layernorm_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ gain,
                                 const int* __restrict__ rows_index, int dim, float eps, float out_scale) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const TX* src = x + (size_t)(rows_index ? rows_index[r] : r) * dim;
    float mean, var;
    row_moments(src, dim, scratch, mean, var);
    const float scale = 1.0f / sqrtf(var + eps);
    TY* dst = y + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = (to_float(src[i]) - mean) * scale * to_float(gain[i]);
        if (out_scale != 1.0f) v *= out_scale;
        if constexpr (ADD) dst[i] = from_float<TY>(to_float(dst[i]) + v);
        else dst[i] = from_float<TY>(v);
    }
}

// y (float32) += norm_a(x); then h = norm_b(y) of the new y (gain_b null: h = the new y itself in h's type).
template <typename TW, typename TH>
__global__ void layernorm_add_norm_kernel(float* __restrict__ y, const float* __restrict__ x, const TW* __restrict__ gain_a,
                                          TH* __restrict__ h, const TW* __restrict__ gain_b, int dim, float eps_a, float eps_b) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t off = (size_t)blockIdx.x * dim;
    const float* src = x + off;
    float* res = y + off;
    TH* dst = h + off;
    float mean, var;
    row_moments(src, dim, scratch, mean, var);
    const float scale_a = 1.0f / sqrtf(var + eps_a);
    float s = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {   // a thread meets the same entries in every loop
        const float v = res[i] + (src[i] - mean) * scale_a * to_float(gain_a[i]);
        res[i] = v;
        s += v;
    }
    if (gain_b == nullptr) {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = from_float<TH>(res[i]);
        return;
    }
    const float mean_b = block_sum(s, scratch) / (float)dim;
    float q = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = res[i] - mean_b;
        q = fmaf(d, d, q);
    }
    const float scale_b = 1.0f / sqrtf(block_sum(q, scratch) / (float)dim + eps_b);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = from_float<TH>((res[i] - mean_b) * scale_b * to_float(gain_b[i]));
}

// The same two kernels for rows of at most PER entries a thread: a thread's entries stay in registers between the passes, so a
// row is read once and the passes do not wait for memory again.
constexpr int LN_PER = 8;

// entry j of a thread's LN_PER: with V = 4 a thread's entries are two runs of four neighbours (16-byte accesses of float32 rows)
template <int V> __device__ __forceinline__ int ln_index(int j) {
    return V == 1 ? (int)(threadIdx.x + j * blockDim.x) : (int)(((j / 4) * blockDim.x + threadIdx.x) * 4 + (j % 4));
}
template <int V> __device__ __forceinline__ void ln_load(const float* __restrict__ src, int dim, float v[LN_PER]) {
    if constexpr (V == 4) {
#pragma unroll
        for (int r = 0; r < LN_PER / 4; r++) {
            const int i = (r * blockDim.x + threadIdx.x) * 4;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < dim) x = *reinterpret_cast<const float4*>(src + i);
            v[4 * r] = x.x; v[4 * r + 1] = x.y; v[4 * r + 2] = x.z; v[4 * r + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < LN_PER; j++) {
            const int i = ln_index<1>(j);
            v[j] = i < dim ? src[i] : 0.f;
        }
    }
}

template <typename TX, typename TW, typename TY, bool ADD, int V = 1>
__global__ void layernorm_cached_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ gain,
                                        const int* __restrict__ rows_index, int dim, float eps, float out_scale) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const TX* src = x + (size_t)(rows_index ? rows_index[r] : r) * dim;
    float v[LN_PER], s = 0.f;
    if constexpr (V == 4) ln_load<4>((const float*)src, dim, v);
    else {
#pragma unroll
        for (int j = 0; j < LN_PER; j++) {
            const int i = ln_index<1>(j);
            v[j] = i < dim ? to_float(src[i]) : 0.f;
        }
    }
#pragma unroll
    for (int j = 0; j < LN_PER; j++) s += v[j];
    const float mean = block_sum(s, scratch) / (float)dim;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < LN_PER; j++) {
        const int i = ln_index<V>(j);
        const float d = i < dim ? v[j] - mean : 0.f;
        q = fmaf(d, d, q);
    }
    const float scale = 1.0f / sqrtf(block_sum(q, scratch) / (float)dim + eps);
    TY* dst = y + (size_t)r * dim;
#pragma unroll
    for (int j = 0; j < LN_PER; j++) {
        const int i = ln_index<V>(j);
        if (i < dim) {
            float o = (v[j] - mean) * scale * to_float(gain[i]);
            if (out_scale != 1.0f) o *= out_scale;
            if constexpr (ADD) dst[i] = from_float<TY>(to_float(dst[i]) + o);
            else dst[i] = from_float<TY>(o);
        }
    }
}

template <typename TW, typename TH, int V = 1>
__global__ void layernorm_add_norm_cached_kernel(float* __restrict__ y, const float* __restrict__ x, const TW* __restrict__ gain_a,
                                                 TH* __restrict__ h, const TW* __restrict__ gain_b, int dim, float eps_a, float eps_b) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t off = (size_t)blockIdx.x * dim;
    float v[LN_PER], old[LN_PER], s = 0.f;
    ln_load<V>(x + off, dim, v);
    ln_load<V>(y + off, dim, old);
#pragma unroll
    for (int j = 0; j < LN_PER; j++) s += v[j];
    const float mean = block_sum(s, scratch) / (float)dim;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < LN_PER; j++) {
        const int i = ln_index<V>(j);
        const float d = i < dim ? v[j] - mean : 0.f;
        q = fmaf(d, d, q);
    }
    const float scale_a = 1.0f / sqrtf(block_sum(q, scratch) / (float)dim + eps_a);
    float s2 = 0.f;
#pragma unroll
    for (int j = 0; j < LN_PER; j++) {
        const int i = ln_index<V>(j);
        if (i < dim) {
            v[j] = old[j] + (v[j] - mean) * scale_a * to_float(gain_a[i]);
            y[off + i] = v[j];
            s2 += v[j];
        }
    }
    if (gain_b == nullptr) {
#pragma unroll
        for (int j = 0; j < LN_PER; j++) {
            const int i = ln_index<V>(j);
            if (i < dim) h[off + i] = from_float<TH>(v[j]);
        }
        return;
    }
    const float mean_b = block_sum(s2, scratch) / (float)dim;
    float q2 = 0.f;
#pragma unroll
    for (int j = 0; j < LN_PER; j++) {
        const int i = ln_index<V>(j);
        const float d = i < dim ? v[j] - mean_b : 0.f;
        q2 = fmaf(d, d, q2);
    }
    const float scale_b = 1.0f / sqrtf(block_sum(q2, scratch) / (float)dim + eps_b);
#pragma unroll
    for (int j = 0; j < LN_PER; j++) {
        const int i = ln_index<V>(j);
        if (i < dim) h[off + i] = from_float<TH>((v[j] - mean_b) * scale_b * to_float(gain_b[i]));
    }
}

// threads of a block whose rows fit LN_PER entries a thread (0: they do not)
inline int cached_threads(int dim) {
    for (int t = 64; t <= 1024; t *= 2)
        if (t * LN_PER >= dim) return t;
    return 0;
}

constexpr int MAX_NORMED_BRANCHES = 4;
struct BranchSumParams {
    const float* x[MAX_NORMED_BRANCHES];
    const void* gain[MAX_NORMED_BRANCHES];
    float scale[MAX_NORMED_BRANCHES];
    float* out;
    int count, dim;
    float eps;
};

template <typename TW>
__global__ void rmsnorm_sum_kernel(BranchSumParams p) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t off = (size_t)blockIdx.x * p.dim;
    float r[MAX_NORMED_BRANCHES];
#pragma unroll
    for (int b = 0; b < MAX_NORMED_BRANCHES; b++) {
        r[b] = 0.f;
        if (b < p.count) {
            const float* src = p.x[b] + off;
            float ss = 0.f;
            for (int i = threadIdx.x; i < p.dim; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
            r[b] = p.scale[b] / sqrtf(block_sum(ss, scratch) / (float)p.dim + p.eps);
        }
    }
    for (int i = threadIdx.x; i < p.dim; i += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int b = 0; b < MAX_NORMED_BRANCHES; b++)
            if (b < p.count) v += p.x[b][off + i] * r[b] * to_float(((const TW*)p.gain[b])[i]);
        p.out[off + i] = v;
    }
}

inline int norm_threads(int dim) { return dim >= 2048 ? 256 : (dim >= 256 ? 128 : (dim >= 64 ? 64 : 32)); }

}  // namespace

HYMT2_API int hymt2_layernorm(void* y, int y_dtype, const void* x, int x_dtype, const void* gain, int gain_dtype, const int* rows_index,
                              int rows, int dim, float eps, float out_scale, int add, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0, "layernorm: bad sizes rows=%d dim=%d", rows, dim);
    HYMT2_REQUIRE(!add || y_dtype == HYMT2_F32, "layernorm: adding into the output needs float32 rows");
    if (const int ct = cached_threads(dim)) {
        if (x_dtype == HYMT2_F32 && dim % 4 == 0 && (uintptr_t)x % 16 == 0 && ct * LN_PER >= dim) {   // 16-byte reads of float32 rows
            HYMT2_DISPATCH_DTYPE(gain_dtype, TW, {
                if (add) {
                    launch_pdl(layernorm_cached_kernel<float, TW, float, true, 4>, dim3(rows), dim3(ct), 0, stream, (float*)y, (const float*)x,
                               (const TW*)gain, rows_index, dim, eps, out_scale);
                } else {
                    HYMT2_DISPATCH_DTYPE(y_dtype, TY, (launch_pdl(layernorm_cached_kernel<float, TW, TY, false, 4>, dim3(rows), dim3(ct), 0, stream,
                                                                  (TY*)y, (const float*)x, (const TW*)gain, rows_index, dim, eps, out_scale)));
                }
            });
            return hymt2_check_launch("layernorm");
        }
        HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(gain_dtype, TW, {
            if (add) {
                launch_pdl(layernorm_cached_kernel<TX, TW, float, true>, dim3(rows), dim3(ct), 0, stream, (float*)y, (const TX*)x, (const TW*)gain,
                           rows_index, dim, eps, out_scale);
            } else {
                HYMT2_DISPATCH_DTYPE(y_dtype, TY, (launch_pdl(layernorm_cached_kernel<TX, TW, TY, false>, dim3(rows), dim3(ct), 0, stream, (TY*)y,
                                                              (const TX*)x, (const TW*)gain, rows_index, dim, eps, out_scale)));
            }
        }));
        return hymt2_check_launch("layernorm");
    }
    const int threads = norm_threads(dim);
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(gain_dtype, TW, {
        if (add) {
            launch_pdl(layernorm_kernel<TX, TW, float, true>, dim3(rows), dim3(threads), 0, stream, (float*)y, (const TX*)x, (const TW*)gain,
                       rows_index, dim, eps, out_scale);
        } else {
            HYMT2_DISPATCH_DTYPE(y_dtype, TY, (launch_pdl(layernorm_kernel<TX, TW, TY, false>, dim3(rows), dim3(threads), 0, stream, (TY*)y,
                                                          (const TX*)x, (const TW*)gain, rows_index, dim, eps, out_scale)));
        }
    }));
    return hymt2_check_launch("layernorm");
}

HYMT2_API int hymt2_layernorm_add_norm(float* y, const float* x, const void* gain_a, void* h, int h_dtype, const void* gain_b, int gain_dtype,
                                       int rows, int dim, float eps_a, float eps_b, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0, "layernorm: bad sizes rows=%d dim=%d", rows, dim);
    if (const int ct = cached_threads(dim)) {
        if (dim % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
            HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(h_dtype, TH,
                (launch_pdl(layernorm_add_norm_cached_kernel<TW, TH, 4>, dim3(rows), dim3(ct), 0, stream, y, x, (const TW*)gain_a, (TH*)h,
                            (const TW*)gain_b, dim, eps_a, eps_b))));
        } else {
            HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(h_dtype, TH,
                (launch_pdl(layernorm_add_norm_cached_kernel<TW, TH>, dim3(rows), dim3(ct), 0, stream, y, x, (const TW*)gain_a, (TH*)h,
                            (const TW*)gain_b, dim, eps_a, eps_b))));
        }
        return hymt2_check_launch("layernorm_add_norm");
    }
    HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(h_dtype, TH,
        (launch_pdl(layernorm_add_norm_kernel<TW, TH>, dim3(rows), dim3(norm_threads(dim)), 0, stream, y, x, (const TW*)gain_a, (TH*)h,
                    (const TW*)gain_b, dim, eps_a, eps_b))));
    return hymt2_check_launch("layernorm_add_norm");
}

HYMT2_API int hymt2_rmsnorm_sum(float* out, const float* const* x, const void* const* gain, const float* scale, int count, int gain_dtype,
                                int rows, int dim, float eps, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0 && count >= 1 && count <= MAX_NORMED_BRANCHES, "rmsnorm_sum: bad sizes rows=%d dim=%d branches=%d",
                  rows, dim, count);
    BranchSumParams p;
    for (int b = 0; b < MAX_NORMED_BRANCHES; b++) {
        p.x[b] = b < count ? x[b] : nullptr;
        p.gain[b] = b < count ? gain[b] : nullptr;
        p.scale[b] = b < count ? scale[b] : 0.f;
    }
    p.out = out; p.count = count; p.dim = dim; p.eps = eps;
    HYMT2_DISPATCH_DTYPE(gain_dtype, TW, launch_pdl(rmsnorm_sum_kernel<TW>, dim3(rows), dim3(norm_threads(dim)), 0, stream, p));
    return hymt2_check_launch("rmsnorm_sum");
}
