// Parts of a layer that carry a small state from token to token: a short causal convolution over time on each
// channel, and the real-gated linear recurrence of a recurrent block.  Both run over the packed tokens of a step
// (sequence b brings the tokens cu_seqlens[b]..cu_seqlens[b+1]-1, the first of them at position kv_lens[b] - n_b)
// and keep their state in the per-sequence state rows of the cache (state + slot * state_stride bytes).
// A sequence whose step starts at position 0 starts from zeros whatever its state row holds.
#include "common.cuh"

namespace {

constexpr int CONV_MAX_TAPS = 16, CONV_CHUNK = 16, CONV_THREADS = 128;

struct ConvParams {
    const void* x;        // [T, ldx] the inputs (channel c of token t at x[t * ldx + c])
    void* out;            // [T, ldo]; must not overlap x
    const float* w;       // [C, taps]; w[c][taps - 1] multiplies the current token
    const float* bias;    // [C] or null
    uint8_t* state;       // state rows; this convolution's part holds float32 [taps - 1][C], oldest first
    long state_stride;    // bytes between two slots' rows
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    int channels, taps, ldx, ldo, add_input;
};

// out_t = act((add_input & 1 ? x_t : 0) + bias + sum_j w[:, j] * x_(t - taps + 1 + j)), zeros before the sequence's start;
// act is SiLU with bit 1 of add_input, else nothing.
// One thread owns a channel over a chunk of a sequence's new tokens and slides a window of registers over it.  The
// thread of the first chunk is the only one that reads the state (for the inputs before this step) and, once it has,
// writes the new one: the last taps - 1 inputs of (old state, new tokens).
template <typename T, int V> struct ChanPack { T v[V]; };
template <typename T, int V> __device__ __forceinline__ void load_chan(const T* p, float out[V]) {
    ChanPack<T, V> r;
    if constexpr (V == 1) r.v[0] = *p;
    else if constexpr (V * sizeof(T) == 4) *reinterpret_cast<uint32_t*>(r.v) = *reinterpret_cast<const uint32_t*>(p);
    else *reinterpret_cast<uint2*>(r.v) = *reinterpret_cast<const uint2*>(p);
#pragma unroll
    for (int k = 0; k < V; k++) out[k] = to_float(r.v[k]);
}
template <typename T, int V> __device__ __forceinline__ void store_chan(T* p, const float in[V]) {
    ChanPack<T, V> r;
#pragma unroll
    for (int k = 0; k < V; k++) r.v[k] = from_float<T>(in[k]);
    if constexpr (V == 1) *p = r.v[0];
    else if constexpr (V * sizeof(T) == 4) *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<const uint32_t*>(r.v);
    else *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(r.v);
}

// A thread owns V neighbouring channels (V = 2 where the rows allow 4- or 8-byte accesses).
template <typename T, int V, int MAXT>
__global__ void __launch_bounds__(CONV_THREADS)
causal_conv_kernel(ConvParams p) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const int c = (blockIdx.x * CONV_THREADS + threadIdx.x) * V;
    const int b = blockIdx.z;
    if (c >= p.channels) return;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    const int i0 = blockIdx.y * CONV_CHUNK;
    if (i0 >= n) return;
    const int slot = p.slot_ids[b];
    const T* x = (const T*)p.x + (size_t)tok0 * p.ldx + c;
    T* out = (T*)p.out + (size_t)tok0 * p.ldo + c;
    const int i1 = min(n, i0 + CONV_CHUNK);
    float zero[V];
#pragma unroll
    for (int k = 0; k < V; k++) zero[k] = 0.f;
    if (slot < 0) {   // a padding row: nothing is remembered, the output is defined
        for (int i = i0; i < i1; i++) store_chan<T, V>(out + (size_t)i * p.ldo, zero);
        return;
    }
    const int start = p.kv_lens[b] - n;   // position of the step's first token
    const int taps = p.taps, hist = taps - 1;
    float* st = (float*)(p.state + (size_t)slot * p.state_stride) + c;   // st[j * channels], j = 0 oldest
    float w[MAXT][V], win[MAXT][V];
#pragma unroll
    for (int j = 0; j < MAXT; j++)
#pragma unroll
        for (int k = 0; k < V; k++) w[j][k] = j < taps ? p.w[(size_t)(c + k) * taps + j] : 0.f;
    // win[j] for j < hist: the input at index i0 - hist + j among the new tokens
#pragma unroll
    for (int j = 0; j < MAXT; j++) {
#pragma unroll
        for (int k = 0; k < V; k++) win[j][k] = 0.f;
        if (j < hist) {
            const int idx = i0 - hist + j;
            if (idx >= 0) load_chan<T, V>(x + (size_t)idx * p.ldx, win[j]);
            else if (start + idx >= 0) {
#pragma unroll
                for (int k = 0; k < V; k++) win[j][k] = st[(size_t)(hist + idx) * p.channels + k];
            }
        }
    }
    float bias[V];
#pragma unroll
    for (int k = 0; k < V; k++) bias[k] = p.bias ? p.bias[c + k] : 0.f;
    for (int i = i0; i < i1; i++) {
        float cur[V], acc[V];
        load_chan<T, V>(x + (size_t)i * p.ldx, cur);
#pragma unroll
        for (int k = 0; k < V; k++) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < MAXT; j++)
                if (j < hist) a = fmaf(w[j][k], win[j][k], a);
#pragma unroll
            for (int j = 0; j < MAXT; j++)
                if (j == hist) a = fmaf(w[j][k], cur[k], a);
            a += bias[k];
            if (p.add_input & 1) a += cur[k];
            if (p.add_input & 2) a = a / (1.0f + expf(-a));   // SiLU of the filter's output
            acc[k] = a;
        }
        store_chan<T, V>(out + (size_t)i * p.ldo, acc);
#pragma unroll
        for (int j = 0; j < MAXT - 1; j++)
            if (j + 1 < hist) {
#pragma unroll
                for (int k = 0; k < V; k++) win[j][k] = win[j + 1][k];
            }
#pragma unroll
        for (int j = 0; j < MAXT; j++)
            if (j == hist - 1) {
#pragma unroll
                for (int k = 0; k < V; k++) win[j][k] = cur[k];
            }
    }
    if (i0 == 0) {
        // new[j] = combined[n + j] of combined = (old state, new tokens); ascending j reads only what is not yet overwritten
        for (int j = 0; j < hist; j++) {
            const int idx = n - hist + j;   // among the new tokens
            float v[V];
#pragma unroll
            for (int k = 0; k < V; k++) v[k] = 0.f;
            if (idx >= 0) load_chan<T, V>(x + (size_t)idx * p.ldx, v);
            else if (start + idx >= 0) {
#pragma unroll
                for (int k = 0; k < V; k++) v[k] = st[(size_t)(hist + idx) * p.channels + k];
            }
#pragma unroll
            for (int k = 0; k < V; k++) st[(size_t)j * p.channels + k] = v[k];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The real-gated linear recurrence.  Per channel c and token t, everything in float32:
//   r = sigmoid(gr + br[c]), i = sigmoid(gi + bi[c])        gr, gi: the gates' sums before their biases
//   log a = -decay * r * softplus(lam[c]);  a = exp(log a)
//   S <- a * S + sqrt(1 - a^2) * i * u;   out = S * y
// One thread owns a channel of one sequence and walks its new tokens in order; the values of RG_BATCH tokens are
// loaded and their coefficients computed side by side, then chained.
// ---------------------------------------------------------------------------------------------------------------
constexpr int RG_BATCH = 8, RG_THREADS = 64;

struct ScanParams {
    const float* gates;   // [T, 2 * width]: gr then gi of every token
    const void* u;        // [T, ldu]
    const void* y;        // [T, ldy]
    void* out;            // [T, ldo]
    const float* br;      // [width]
    const float* bi;      // [width]
    const float* lam;     // [width]
    uint8_t* state;
    long state_stride;
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    int width, ldu, ldy, ldo;
    float decay;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// Walks tokens [i_begin, i_end) of one sequence's channel c from the state S; returns the new S.  WRITE: the outputs
// S * y are stored; otherwise only the state moves (and *prod collects the product of the decays on the way).
template <typename T, bool WRITE>
__device__ __forceinline__ float rglru_walk(const ScanParams& p, int c, int tok0, int i_begin, int i_end, float S, float* prod) {
    const float br = p.br[c], bi = p.bi[c];
    const float rate = -p.decay * softplus_f(p.lam[c]);
    const float* gates = p.gates + (size_t)tok0 * 2 * p.width + c;
    const T* u = (const T*)p.u + (size_t)tok0 * p.ldu + c;
    const T* y = (const T*)p.y + (size_t)tok0 * p.ldy + c;
    T* out = (T*)p.out + (size_t)tok0 * p.ldo + c;
    float A = 1.f;
    for (int i0 = i_begin; i0 < i_end; i0 += RG_BATCH) {
        float a[RG_BATCH], bx[RG_BATCH], yy[RG_BATCH];
#pragma unroll
        for (int k = 0; k < RG_BATCH; k++) {
            const int i = i0 + k;
            a[k] = 1.f; bx[k] = 0.f; yy[k] = 0.f;
            if (i < i_end) {
                const float r = sigmoid_f(gates[(size_t)i * 2 * p.width] + br);
                const float g = sigmoid_f(gates[(size_t)i * 2 * p.width + p.width] + bi);
                const float log_a = rate * r;
                a[k] = expf(log_a);
                bx[k] = sqrtf(-expm1f(2.f * log_a)) * g * to_float(u[(size_t)i * p.ldu]);
                if (WRITE) yy[k] = to_float(y[(size_t)i * p.ldy]);
            }
        }
#pragma unroll
        for (int k = 0; k < RG_BATCH; k++) {
            const int i = i0 + k;
            if (i < i_end) {
                S = fmaf(a[k], S, bx[k]);
                A *= a[k];
                if (WRITE) out[(size_t)i * p.ldo] = from_float<T>(S * yy[k]);
            }
        }
    }
    if (prod) *prod = A;
    return S;
}

// One thread walks ALL new tokens of its sequence's channel: decode steps and short portions.
template <typename T>
__global__ void __launch_bounds__(RG_THREADS)
rglru_scan_kernel(ScanParams p) {
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const int c = blockIdx.x * RG_THREADS + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= p.width) return;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    const int slot = p.slot_ids[b];
    if (slot < 0) {
        T* out = (T*)p.out + (size_t)tok0 * p.ldo + c;
        for (int i = 0; i < n; i++) out[(size_t)i * p.ldo] = from_float<T>(0.f);
        return;
    }
    const int start = p.kv_lens[b] - n;
    float* st = (float*)(p.state + (size_t)slot * p.state_stride) + c;
    *st = rglru_walk<T, true>(p, c, tok0, 0, n, start > 0 ? *st : 0.f, nullptr);
}

// Long portions in two passes over chunks of RG_CHUNK tokens.  The recurrence S <- a S + b composes: a chunk as a whole
// is S_out = A * S_in + B with A the product of its decays and B what it leaves from a zero state.  Pass 1: every
// (chunk, channel) thread finds its (A, B); the threads of chunk 0 also note the state that the sequence came with.
// Pass 2: every thread folds the (A, B) of the chunks before its own, in order, into its S_in, walks its chunk again
// and writes the outputs; the last chunk's thread leaves the new state.
// scratch: [batch][chunks + 1][2][width] floats; entry `chunks` holds the incoming state.
constexpr int RG_CHUNK = 64;

template <typename T, int PASS>
__global__ void __launch_bounds__(RG_THREADS)
rglru_chunk_kernel(ScanParams p, float* scratch, int chunks) {
    const int c = blockIdx.x * RG_THREADS + threadIdx.x;
    const int k = blockIdx.y, b = blockIdx.z;
    if (c >= p.width) return;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    const int i0 = k * RG_CHUNK;
    if (i0 >= n) return;
    const int i1 = min(n, i0 + RG_CHUNK);
    const int slot = p.slot_ids[b];
    float* mine = scratch + ((size_t)b * (chunks + 1)) * 2 * p.width + c;
    if (slot < 0) {
        if (PASS == 2) {
            T* out = (T*)p.out + (size_t)tok0 * p.ldo + c;
            for (int i = i0; i < i1; i++) out[(size_t)i * p.ldo] = from_float<T>(0.f);
        }
        return;
    }
    float* st = (float*)(p.state + (size_t)slot * p.state_stride) + c;
    if (PASS == 1) {
        float A;
        const float B = rglru_walk<T, false>(p, c, tok0, i0, i1, 0.f, &A);
        mine[(size_t)k * 2 * p.width] = A;
        mine[(size_t)k * 2 * p.width + p.width] = B;
        if (k == 0) mine[(size_t)chunks * 2 * p.width] = p.kv_lens[b] - n > 0 ? *st : 0.f;
    } else {
        float S = mine[(size_t)chunks * 2 * p.width];
        for (int j = 0; j < k; j++) S = fmaf(mine[(size_t)j * 2 * p.width], S, mine[(size_t)j * 2 * p.width + p.width]);
        S = rglru_walk<T, true>(p, c, tok0, i0, i1, S, nullptr);
        if (i1 == n) *st = S;
    }
}

}  // namespace

HYMT2_API int hymt2_causal_conv(void* out, const void* x, int dtype, const float* w, const float* bias, void* state,
                                long state_offset, long state_stride, const int* cu_seqlens, const int* slot_ids,
                                const int* kv_lens, int batch, int max_new_tokens, int channels, int taps, int ldx, int ldo,
                                int add_input, cudaStream_t stream) {
    if (batch == 0 || max_new_tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && channels > 0 && max_new_tokens > 0, "causal_conv: bad sizes");
    HYMT2_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: %d taps; 1 to %d are taken", taps, CONV_MAX_TAPS);
    HYMT2_REQUIRE(state_offset % 4 == 0 && state_stride % 4 == 0, "causal_conv: the state must be 4-byte aligned");
    HYMT2_REQUIRE(ldx >= channels && ldo >= channels, "causal_conv: a row is shorter than the channels");
    ConvParams p;
    p.x = x; p.out = out; p.w = w; p.bias = bias; p.state = (uint8_t*)state + state_offset; p.state_stride = state_stride;
    p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.channels = channels; p.taps = taps; p.ldx = ldx; p.ldo = ldo; p.add_input = add_input;
    const int chunks = (max_new_tokens + CONV_CHUNK - 1) / CONV_CHUNK;
    HYMT2_REQUIRE(chunks <= 65535, "causal_conv: %d tokens in one sequence are too many for one launch", max_new_tokens);
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        const bool pairs = channels % 2 == 0 && ldx % 2 == 0 && ldo % 2 == 0 && (uintptr_t)x % (2 * sizeof(T)) == 0 && (uintptr_t)out % (2 * sizeof(T)) == 0;
        // (the window of inputs lives in registers: a kernel for filters of up to 4 taps, one for up to 16)
        if (pairs) {
            const dim3 grid((channels / 2 + CONV_THREADS - 1) / CONV_THREADS, chunks, batch);
            if (taps <= 4) launch_pdl(causal_conv_kernel<T, 2, 4>, grid, dim3(CONV_THREADS), 0, stream, p);
            else launch_pdl(causal_conv_kernel<T, 2, CONV_MAX_TAPS>, grid, dim3(CONV_THREADS), 0, stream, p);
        } else {
            const dim3 grid((channels + CONV_THREADS - 1) / CONV_THREADS, chunks, batch);
            if (taps <= 4) launch_pdl(causal_conv_kernel<T, 1, 4>, grid, dim3(CONV_THREADS), 0, stream, p);
            else launch_pdl(causal_conv_kernel<T, 1, CONV_MAX_TAPS>, grid, dim3(CONV_THREADS), 0, stream, p);
        }
    });
    return hymt2_check_launch("causal_conv");
}

// Floats of scratch that a step whose longest portion has max_new_tokens tokens needs (0: one pass, no scratch).
HYMT2_API long hymt2_rglru_scan_scratch(int batch, int max_new_tokens, int width) {
    if (max_new_tokens <= 2 * RG_CHUNK) return 0;
    const long chunks = (max_new_tokens + RG_CHUNK - 1) / RG_CHUNK;
    return (long)batch * (chunks + 1) * 2 * width;
}

HYMT2_API int hymt2_rglru_scan(void* out, const float* gates, const void* u, const void* y, int dtype, const float* br,
                               const float* bi, const float* lam, float decay, void* state, long state_offset,
                               long state_stride, const int* cu_seqlens, const int* slot_ids, const int* kv_lens, int batch,
                               int width, int ldu, int ldy, int ldo, int max_new_tokens, float* scratch, long scratch_floats,
                               cudaStream_t stream) {
    if (batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && width > 0, "rglru_scan: bad sizes");
    HYMT2_REQUIRE(state_offset % 4 == 0 && state_stride % 4 == 0, "rglru_scan: the state must be 4-byte aligned");
    ScanParams p;
    p.gates = gates; p.u = u; p.y = y; p.out = out; p.br = br; p.bi = bi; p.lam = lam;
    p.state = (uint8_t*)state + state_offset; p.state_stride = state_stride;
    p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.width = width; p.ldu = ldu; p.ldy = ldy; p.ldo = ldo; p.decay = decay;
    const long need = hymt2_rglru_scan_scratch(batch, max_new_tokens, width);
    if (need > 0) {
        HYMT2_REQUIRE(scratch != nullptr && scratch_floats >= need, "rglru_scan: %ld floats of scratch are needed", need);
        const int chunks = (max_new_tokens + RG_CHUNK - 1) / RG_CHUNK;
        HYMT2_REQUIRE(chunks <= 65535, "rglru_scan: %d tokens in one portion are too many", max_new_tokens);
        const dim3 grid((width + RG_THREADS - 1) / RG_THREADS, chunks, batch);
        HYMT2_DISPATCH_DTYPE(dtype, T, {
            rglru_chunk_kernel<T, 1><<<grid, RG_THREADS, 0, stream>>>(p, scratch, chunks);
            rglru_chunk_kernel<T, 2><<<grid, RG_THREADS, 0, stream>>>(p, scratch, chunks);
        });
        return hymt2_check_launch("rglru_scan");
    }
    const dim3 grid((width + RG_THREADS - 1) / RG_THREADS, batch);
    HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(rglru_scan_kernel<T>, grid, dim3(RG_THREADS), 0, stream, p));
    return hymt2_check_launch("rglru_scan");
}
