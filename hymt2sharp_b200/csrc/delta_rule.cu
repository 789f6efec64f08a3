// The gated delta rule: a recurrence over a matrix of state S [dk, dv] float32 per (sequence, value head), with one decay per
// token, head and key channel and a write that first takes away what the state already answers for the key:
//
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          (the read sees the write)
//
// `delta_prep` makes what enters the recurrence, all in float32, from what the projections and the short convolutions left:
// q and k of every key head as unit vectors x / sqrt(sum(x^2) + unit_eps) (q also times q_scale), the decays
// g = exp(-exp(A_log[h]) * softplus(x + dt_bias)) in place of x, and beta = sigmoid(.) in place.
// `delta_scan` walks a sequence's new tokens.  The columns of S never meet (u's entry c needs column c only), so the grid
// spreads them: a block holds COLS columns of one (sequence, head), TPC neighbouring lanes share a column and hold RPT of its
// rows each in registers (dk <= RPT * TPC); the two sums over rows are finished with shuffles inside the TPC lanes.  The next
// token's k, q and g are fetched while the current token is worked on.  S lies at byte `state_offset` of the sequence's state
// row as [heads, dk, dv]; a sequence whose step starts at position 0 starts from zeros whatever the row holds; a padding row
// (slot < 0) writes zeros and remembers nothing.
#include "common.cuh"

namespace {

struct DeltaPrepParams {
    const void* qk;       // [T, ldqk]: q of all key heads [kv_heads * dk], then k the same
    float* qn;            // [T, kv_heads * dk]
    float* kn;
    float* decay;         // [T, heads * dk]: in x, out g
    float* beta;          // [T, ldb]: in the projection, out its sigmoid
    const float* dt_bias; // [heads * dk]
    const float* a_log;   // [heads]
    long ldqk, ldb;
    int heads, kv_heads, dk;
    float q_scale, unit_eps;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(128)
delta_prep_kernel(DeltaPrepParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* row = (const T*)p.qk + (size_t)t * p.ldqk;
    const int kd = p.kv_heads * p.dk;
    for (int item = warp; item < 2 * p.kv_heads; item += 4) {     // (q or k, key head)
        const bool is_k = item >= p.kv_heads;
        const int g = is_k ? item - p.kv_heads : item;
        const T* src = row + (is_k ? kd : 0) + (size_t)g * p.dk;
        float ss = 0.f;
        for (int i = lane; i < p.dk; i += 32) {
            const float v = to_float(src[i]);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float r = (is_k ? 1.0f : p.q_scale) / sqrtf(ss + p.unit_eps);
        float* dst = (is_k ? p.kn : p.qn) + (size_t)t * kd + (size_t)g * p.dk;
        for (int i = lane; i < p.dk; i += 32) dst[i] = to_float(src[i]) * r;
    }
    const int hd = p.heads * p.dk;
    float* dec = p.decay + (size_t)t * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        const float rate = expf(p.a_log[i / p.dk]);
        dec[i] = expf(-rate * softplus_f(dec[i] + p.dt_bias[i]));
    }
    for (int i = threadIdx.x; i < p.heads; i += blockDim.x) {
        float* b = p.beta + (size_t)t * p.ldb + i;
        *b = 1.0f / (1.0f + expf(-*b));
    }
}

struct DeltaScanParams {
    float* out;            // [T, heads * dv]
    const float* q;        // [T, kv_heads * dk] unit vectors (q scaled)
    const float* k;
    const float* decay;    // [T, heads * dk]
    const float* beta;     // [T, ldb]
    const void* v;         // [T, ldv] compute type
    uint8_t* state;
    long state_stride, ldv, ldb;
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    int heads, kv_heads, dk, dv;
};

template <int TPC> __device__ __forceinline__ float part_sum(float v) {
#pragma unroll
    for (int o = TPC / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int DELTA_THREADS = 64;

template <typename T, int RPT, int TPC>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_scan_kernel(DeltaScanParams p) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int COLS = DELTA_THREADS / TPC;
    const int b = blockIdx.z, h = blockIdx.y;
    const int c = blockIdx.x * COLS + threadIdx.x / TPC, part = threadIdx.x % TPC;
    const bool live = c < p.dv;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    if (n <= 0) return;
    const int slot = p.slot_ids[b];
    const int hd = p.heads * p.dv;
    if (slot < 0) {
        if (live && part == 0)
            for (int i = 0; i < n; i++) p.out[(size_t)(tok0 + i) * hd + (size_t)h * p.dv + c] = 0.f;
        return;
    }
    const int start = p.kv_lens[b] - n;
    const int kh = h / (p.heads / p.kv_heads);
    const int r0 = part * RPT;
    float* S = (float*)(p.state + (size_t)slot * p.state_stride) + (size_t)h * p.dk * p.dv;
    float s[RPT];
#pragma unroll
    for (int i = 0; i < RPT; i++) s[i] = (start > 0 && live && r0 + i < p.dk) ? S[(size_t)(r0 + i) * p.dv + c] : 0.f;
    const size_t kd = (size_t)p.kv_heads * p.dk, gd = (size_t)p.heads * p.dk;
    const float* kp = p.k + (size_t)tok0 * kd + (size_t)kh * p.dk + r0;
    const float* qp = p.q + (size_t)tok0 * kd + (size_t)kh * p.dk + r0;
    const float* gp = p.decay + (size_t)tok0 * gd + (size_t)h * p.dk + r0;
    float nk[RPT], nq[RPT], ng[RPT], nb, nv;
    auto fetch = [&](int i) {
#pragma unroll
        for (int j = 0; j < RPT; j++) {
            const bool in = r0 + j < p.dk;
            nk[j] = in ? kp[(size_t)i * kd + j] : 0.f;
            nq[j] = in ? qp[(size_t)i * kd + j] : 0.f;
            ng[j] = in ? gp[(size_t)i * gd + j] : 1.f;
        }
        nb = p.beta[(size_t)(tok0 + i) * p.ldb + h];
        nv = live ? to_float(((const T*)p.v)[(size_t)(tok0 + i) * p.ldv + (size_t)h * p.dv + c]) : 0.f;
    };
    fetch(0);
    for (int i = 0; i < n; i++) {
        float k[RPT], q[RPT], g[RPT];
#pragma unroll
        for (int j = 0; j < RPT; j++) { k[j] = nk[j]; q[j] = nq[j]; g[j] = ng[j]; }
        const float beta = nb, v = nv;
        if (i + 1 < n) fetch(i + 1);
        float pred = 0.f;
#pragma unroll
        for (int j = 0; j < RPT; j++) {
            s[j] *= g[j];
            pred = fmaf(s[j], k[j], pred);
        }
        pred = part_sum<TPC>(pred);
        const float u = beta * (v - pred);
        float o = 0.f;
#pragma unroll
        for (int j = 0; j < RPT; j++) {
            s[j] = fmaf(k[j], u, s[j]);
            o = fmaf(s[j], q[j], o);
        }
        o = part_sum<TPC>(o);
        if (live && part == 0) p.out[(size_t)(tok0 + i) * hd + (size_t)h * p.dv + c] = o;
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < RPT; j++)
            if (r0 + j < p.dk) S[(size_t)(r0 + j) * p.dv + c] = s[j];
    }
}

}  // namespace

HYMT2_API int hymt2_delta_prep(const void* qk, long ldqk, int dtype, float* qn, float* kn, float* decay, float* beta, long ldb,
                               const float* dt_bias, const float* a_log, int tokens, int heads, int kv_heads, int dk, float q_scale,
                               float unit_eps, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0, "delta_prep: bad sizes");
    DeltaPrepParams p;
    p.qk = qk; p.qn = qn; p.kn = kn; p.decay = decay; p.beta = beta; p.dt_bias = dt_bias; p.a_log = a_log; p.ldqk = ldqk; p.ldb = ldb;
    p.heads = heads; p.kv_heads = kv_heads; p.dk = dk; p.q_scale = q_scale; p.unit_eps = unit_eps;
    HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(delta_prep_kernel<T>, dim3(tokens), dim3(128), 0, stream, p));
    return hymt2_check_launch("delta_prep");
}

HYMT2_API int hymt2_delta_scan_max_dk() { return 256; }

HYMT2_API int hymt2_delta_scan(float* out, const float* q, const float* k, const float* decay, const float* beta, long ldb, const void* v,
                               long ldv, int dtype, void* state, long state_offset, long state_stride, const int* cu_seqlens,
                               const int* slot_ids, const int* kv_lens, int batch, int heads, int kv_heads, int dk, int dv,
                               cudaStream_t stream) {
    if (batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && heads > 0 && heads <= 65535 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0,
                  "delta_scan: bad sizes");
    HYMT2_REQUIRE(dk <= 256, "delta_scan: %d key channels a head; up to 256 are taken", dk);
    HYMT2_REQUIRE(state_offset % 4 == 0 && state_stride % 4 == 0, "delta_scan: the state must be 4-byte aligned");
    DeltaScanParams p;
    p.out = out; p.q = q; p.k = k; p.decay = decay; p.beta = beta; p.v = v; p.state = (uint8_t*)state + state_offset;
    p.state_stride = state_stride; p.ldv = ldv; p.ldb = ldb; p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.heads = heads; p.kv_heads = kv_heads; p.dk = dk; p.dv = dv;
#define DELTA_LAUNCH(RPT, TPC)                                                                                             \
    do {                                                                                                                   \
        const dim3 grid((dv + DELTA_THREADS / TPC - 1) / (DELTA_THREADS / TPC), heads, batch);                             \
        HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(delta_scan_kernel<T, RPT, TPC>, grid, dim3(DELTA_THREADS), 0, stream, p)); \
    } while (0)
    if (dk <= 16) DELTA_LAUNCH(4, 4);
    else if (dk <= 32) DELTA_LAUNCH(8, 4);
    else if (dk <= 64) DELTA_LAUNCH(16, 4);
    else if (dk <= 128) DELTA_LAUNCH(32, 4);
    else DELTA_LAUNCH(32, 8);
#undef DELTA_LAUNCH
    return hymt2_check_launch("delta_scan");
}
