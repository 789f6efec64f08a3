// A residual that is kept as several streams (hyper-connections).  X is float32 [streams, tokens, width]; a sublayer
// reads one mixture of the streams and its output is written back into all of them:
//
//   read    u[t] = sum_s w_in[s] X[s][t];  out[t] = u[t] / sqrt(mean(u[t]^2) + eps) * gain   (without a gain: out = u, float32)
//   write   y[t] = sum_b scale_b * branch_b[t];  X'[r][t] = sum_s mix[s][r] X[s][t] + w_out[r] * y[t], every r from the OLD streams
//   write_read   the write, and the read of the sublayer that comes next, of the new streams, in one pass over a token's row
//   fill    X[s] = X[0] for every s > 0
//
// Everything is float32; a sum over streams runs in ascending s, a sum over branches in ascending b.  One block per token.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8, MAX_BRANCHES = 4, THREADS = 256;

struct StreamsParams {
    float* X;                 // [streams][tokens][width]
    const float* w_in;        // [streams] of the read (may be null: no read)
    const float* mix;         // [streams][streams], indexed [from][to] (null: no write)
    const float* w_out;       // [streams]
    const float* branch[MAX_BRANCHES];
    float scale[MAX_BRANCHES];
    int branches;
    const void* gain;         // [width] or null
    void* out;                // [tokens][width]
    int streams, tokens, width;
    float eps;
};

// V columns a thread and access (4 where the width and the addresses allow 16-byte accesses, else 1); SM: the most streams that
// the instance holds in registers (2, 4 or MAX_STREAMS: the fewer, the more blocks an SM keeps in flight).
template <typename TO, typename TG, bool WRITE, bool READ, int V, int SM>
__global__ void __launch_bounds__(THREADS)
streams_kernel(StreamsParams p) {
    __shared__ float scratch[33];
    __shared__ float s_in[MAX_STREAMS], s_out[MAX_STREAMS], s_mix[MAX_STREAMS * MAX_STREAMS];
    const int S = p.streams, W = p.width;
    if (threadIdx.x < S) {                                  // the small tables never depend on the kernel in front
        if (READ) s_in[threadIdx.x] = p.w_in[threadIdx.x];
        if (WRITE) s_out[threadIdx.x] = p.w_out[threadIdx.x];
    }
    if (WRITE && threadIdx.x < S * S) s_mix[threadIdx.x] = p.mix[threadIdx.x];
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    const size_t t = blockIdx.x;
    const size_t plane = (size_t)p.tokens * W;
    float* row = p.X + t * W;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < W; c += THREADS * V) {
        Pack<float, V> x[SM];
#pragma unroll
        for (int s = 0; s < SM; s++)
            if (s < S) x[s] = load_pack<float, V>(row + s * plane + c);
        if (WRITE) {
            Pack<float, V> y;
#pragma unroll
            for (int e = 0; e < V; e++) y.v[e] = 0.f;
#pragma unroll
            for (int b = 0; b < MAX_BRANCHES; b++)
                if (b < p.branches) {
                    const Pack<float, V> br = load_pack<float, V>(p.branch[b] + t * W + c);
#pragma unroll
                    for (int e = 0; e < V; e++) y.v[e] = fmaf(p.scale[b], br.v[e], y.v[e]);
                }
            Pack<float, V> nx[SM];
#pragma unroll
            for (int r = 0; r < SM; r++) {
                if (r >= S) continue;
#pragma unroll
                for (int e = 0; e < V; e++) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < SM; s++)
                        if (s < S) a = fmaf(s_mix[s * S + r], x[s].v[e], a);
                    nx[r].v[e] = fmaf(s_out[r], y.v[e], a);
                }
                store_pack<float, V>(row + r * plane + c, nx[r]);
            }
#pragma unroll
            for (int s = 0; s < SM; s++)
                if (s < S) x[s] = nx[s];
        }
        if (READ) {
            Pack<float, V> u;
#pragma unroll
            for (int e = 0; e < V; e++) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < SM; s++)
                    if (s < S) a = fmaf(s_in[s], x[s].v[e], a);
                u.v[e] = a;
                ss = fmaf(a, a, ss);
            }
            if (p.gain == nullptr) store_pack<float, V>((float*)p.out + t * W + c, u);
        }
    }
    if (!READ || p.gain == nullptr) return;
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)W + p.eps);
    // the same thread wrote the entries that it reads here again
    for (int c = threadIdx.x * V; c < W; c += THREADS * V) {
        Pack<float, V> u;
#pragma unroll
        for (int e = 0; e < V; e++) u.v[e] = 0.f;
#pragma unroll
        for (int s = 0; s < SM; s++)
            if (s < S) {
                const Pack<float, V> xs = load_pack<float, V>(row + s * plane + c);
#pragma unroll
                for (int e = 0; e < V; e++) u.v[e] = fmaf(s_in[s], xs.v[e], u.v[e]);
            }
        const Pack<TG, V> g = load_pack<TG, V>((const TG*)p.gain + c);
        Pack<TO, V> o;
#pragma unroll
        for (int e = 0; e < V; e++) o.v[e] = from_float<TO>(u.v[e] * r * to_float(g.v[e]));
        store_pack<TO, V>((TO*)p.out + t * W + c, o);
    }
}

__global__ void __launch_bounds__(256)
streams_fill_kernel(float4* X, size_t plane4, int streams) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= plane4) return;
    const float4 v = X[i];
    for (int s = 1; s < streams; s++) X[s * plane4 + i] = v;
}

__global__ void __launch_bounds__(256)
streams_fill_scalar_kernel(float* X, size_t plane, int streams) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= plane) return;
    const float v = X[i];
    for (int s = 1; s < streams; s++) X[s * plane + i] = v;
}

}  // namespace

HYMT2_API int hymt2_streams_fill(float* X, int streams, int tokens, int width, cudaStream_t stream) {
    if (tokens == 0 || streams <= 1) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && width > 0, "streams_fill: bad sizes");
    const size_t plane = (size_t)tokens * width;
    if (plane % 4 == 0 && (uintptr_t)X % 16 == 0)
        launch_pdl(streams_fill_kernel, dim3((unsigned)((plane / 4 + 255) / 256)), dim3(256), 0, stream, (float4*)X, plane / 4, streams);
    else
        launch_pdl(streams_fill_scalar_kernel, dim3((unsigned)((plane + 255) / 256)), dim3(256), 0, stream, X, plane, streams);
    return hymt2_check_launch("streams_fill");
}

// Any of the three forms: write (mix != null), read (w_in != null), or both.  `branches` point to float32 [tokens, width].
HYMT2_API int hymt2_streams_step(float* X, int streams, int tokens, int width, const float* mix, const float* w_out,
                                 const float* const* branches, const float* scales, int num_branches, const float* w_in,
                                 const void* gain, int gain_dtype, float eps, void* out, int out_dtype, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && width > 0 && streams > 0 && streams <= MAX_STREAMS, "streams: %d streams (at most %d)", streams, MAX_STREAMS);
    const bool write = mix != nullptr, read = w_in != nullptr;
    HYMT2_REQUIRE(write || read, "streams: nothing to do");
    HYMT2_REQUIRE(!write || (w_out && num_branches > 0 && num_branches <= MAX_BRANCHES), "streams: a write needs 1 to %d branches", MAX_BRANCHES);
    HYMT2_REQUIRE(!read || out, "streams: a read needs a place for its rows");
    HYMT2_REQUIRE(!read || gain || out_dtype == HYMT2_F32, "streams: a read without a norm gives float32 rows");
    StreamsParams p{};
    p.X = X; p.w_in = w_in; p.mix = mix; p.w_out = w_out; p.branches = write ? num_branches : 0;
    for (int b = 0; b < p.branches; b++) { p.branch[b] = branches[b]; p.scale[b] = scales[b]; }
    p.gain = gain; p.out = out; p.streams = streams; p.tokens = tokens; p.width = width; p.eps = eps;
    if (!gain) gain_dtype = HYMT2_F32;
    // 16-byte accesses: the width a multiple of 4 (rows and planes then start on multiples of 4 entries) and every base aligned
    bool wide = width % 4 == 0 && (uintptr_t)X % 16 == 0 && (!out || (uintptr_t)out % 16 == 0) && (!gain || (uintptr_t)gain % 16 == 0);
    for (int b = 0; b < p.branches; b++) wide = wide && (uintptr_t)p.branch[b] % 16 == 0;
#define HYMT2_STREAMS_LAUNCH(V, SM)                                                                                               \
    do {                                                                                                                          \
        if (write && read) launch_pdl(streams_kernel<TO, TG, true, true, V, SM>, dim3(tokens), dim3(THREADS), 0, stream, p);      \
        else if (write) launch_pdl(streams_kernel<TO, TG, true, false, V, SM>, dim3(tokens), dim3(THREADS), 0, stream, p);        \
        else launch_pdl(streams_kernel<TO, TG, false, true, V, SM>, dim3(tokens), dim3(THREADS), 0, stream, p);                   \
    } while (0)
    HYMT2_DISPATCH_DTYPE(out_dtype, TO, HYMT2_DISPATCH_DTYPE(gain_dtype, TG, {
        if (wide) {
            if (streams <= 2) HYMT2_STREAMS_LAUNCH(4, 2);
            else if (streams <= 4) HYMT2_STREAMS_LAUNCH(4, 4);
            else HYMT2_STREAMS_LAUNCH(4, MAX_STREAMS);
        } else {
            if (streams <= 2) HYMT2_STREAMS_LAUNCH(1, 2);
            else if (streams <= 4) HYMT2_STREAMS_LAUNCH(1, 4);
            else HYMT2_STREAMS_LAUNCH(1, MAX_STREAMS);
        }
    }));
#undef HYMT2_STREAMS_LAUNCH
    return hymt2_check_launch("streams_step");
}
