// The gated delta rule: a recurrence over a matrix of state S [dk, dv] float32 per (sequence, value head), with one decay per
// token, head and key channel and a write that first takes away what the state already answers for the key:
//
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          (the read sees the write)
//
// `delta_prep` makes what enters the recurrence, all in float32, from what the projections and the short convolutions left:
// q and k of every key head as unit vectors x / sqrt(sum(x^2) + unit_eps) (q also times q_scale), the decays
// g = exp(-exp(A_log[h]) * softplus(x + dt_bias)) in place of x, and beta = sigmoid(.) in place.
// `delta_scan` walks a sequence's new tokens.  The columns of S never meet (u's entry c needs column c only), so the grid
// spreads them: a block holds 16 columns of one (sequence, head), 8 neighbouring lanes share a column and hold RPT of its
// rows each in registers (dk <= 8 * RPT); the two sums over rows are finished with shuffles inside those lanes.  The tokens'
// vectors are staged through shared memory a group at a time, the next group being fetched while the current one is worked on.
// S lies at byte `state_offset` of the sequence's state row as [heads, dk, dv]; a sequence whose step starts at position 0 starts from zeros whatever the row holds; a padding row
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
    // (the blocks of a token share its work among themselves: blockIdx.y of gridDim.y)
    const int share = blockIdx.y, shares = gridDim.y;
    for (int item = warp + 4 * share; item < 2 * p.kv_heads; item += 4 * shares) {     // (q or k, key head)
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
    for (int i = threadIdx.x + share * blockDim.x; i < hd; i += blockDim.x * shares) {
        const float rate = expf(p.a_log[i / p.dk]);
        dec[i] = expf(-rate * softplus_f(dec[i] + p.dt_bias[i]));
    }
    for (int i = threadIdx.x + share * blockDim.x; i < p.heads; i += blockDim.x * shares) {
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

constexpr int DELTA_THREADS = 128, DELTA_TPC = 8, DELTA_COLS = DELTA_THREADS / DELTA_TPC;

__device__ __forceinline__ float part_sum(float v) {
#pragma unroll
    for (int o = DELTA_TPC / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// A block holds DELTA_COLS columns of one (sequence, head)'s state; DELTA_TPC neighbouring lanes share a column and hold RPT of
// its rows each in registers (dk <= DKP = RPT * DELTA_TPC; rows beyond dk are k = q = 0, g = 1 and stay zero).  The tokens' k, q,
// g (float32), beta and the block's entries of v are staged through shared memory in groups of DELTA_GROUP tokens: while a group
// is worked on, the next one is already on its way from global memory into registers.  Steps of one token a sequence take the
// instance with groups of one: a fraction of the registers, so that many more blocks stream their states at once.
template <typename T, int RPT, int DELTA_GROUP>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_scan_kernel(DeltaScanParams p) {
    constexpr int DKP = RPT * DELTA_TPC;
    constexpr int TOKEN = 3 * DKP + DELTA_COLS + 4;                    // staged floats a token: k, q, g, the block's v, beta (and three unused: 16-byte rows)
    constexpr int ITEMS = DELTA_GROUP * TOKEN;
    __shared__ __align__(16) float stage[ITEMS];
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.z, h = blockIdx.y;
    const int c0 = blockIdx.x * DELTA_COLS;
    const int col = threadIdx.x / DELTA_TPC, part = threadIdx.x % DELTA_TPC;
    const int c = c0 + col;
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
    for (int j = 0; j < RPT; j++) s[j] = (start > 0 && live && r0 + j < p.dk) ? S[(size_t)(r0 + j) * p.dv + c] : 0.f;
    const size_t kd = (size_t)p.kv_heads * p.dk, gd = (size_t)p.heads * p.dk;
    const float* kp = p.k + (size_t)tok0 * kd + (size_t)kh * p.dk;
    const float* qp = p.q + (size_t)tok0 * kd + (size_t)kh * p.dk;
    const float* gp = p.decay + (size_t)tok0 * gd + (size_t)h * p.dk;
    const T* vp = (const T*)p.v + (size_t)tok0 * p.ldv + (size_t)h * p.dv + c0;
    const float* bp = p.beta + (size_t)tok0 * p.ldb + h;
    // Staging: thread t brings rows t, t + 128, ... of k, q and g of each of the group's tokens, one of the group's entries of v
    // (token t / 16, column t % 16) and, the first eight threads, a token's beta.  A token behind the sequence's end is one that
    // changes nothing (k = q = v = beta = 0, g = 1), so that a group is always walked whole; rows beyond dk the same.
    // In shared memory the rows of k, q, g are interleaved so that the eight lanes of a column read their j-th four rows from
    // eight neighbouring 16-byte pieces (row r = part * RPT + 4 j + x -> piece j * 8 + part, entry x).
    static_assert(DELTA_GROUP * DELTA_COLS <= DELTA_THREADS, "at most one entry of v a thread");
    constexpr int RP = (DKP + DELTA_THREADS - 1) / DELTA_THREADS;
    int place[RP];
#pragma unroll
    for (int x = 0; x < RP; x++) {
        const int r = threadIdx.x + x * DELTA_THREADS;
        place[x] = (((r % RPT) / 4) * DELTA_TPC + r / RPT) * 4 + (r % 4);
    }
    const int vt = threadIdx.x / DELTA_COLS, vc = threadIdx.x % DELTA_COLS;
    float pre[DELTA_GROUP][3][RP], pre_v, pre_b;
    auto fetch = [&](int i0) {
#pragma unroll
        for (int tt = 0; tt < DELTA_GROUP; tt++) {
            const int i = i0 + tt;
#pragma unroll
            for (int x = 0; x < RP; x++) {
                const int r = threadIdx.x + x * DELTA_THREADS;
                const bool in = i < n && r < p.dk;
                pre[tt][0][x] = in ? kp[(size_t)i * kd + r] : 0.f;
                pre[tt][1][x] = in ? qp[(size_t)i * kd + r] : 0.f;
                pre[tt][2][x] = in ? gp[(size_t)i * gd + r] : 1.f;
            }
        }
        pre_v = (vt < DELTA_GROUP && i0 + vt < n && c0 + vc < p.dv) ? to_float(vp[(size_t)(i0 + vt) * p.ldv + vc]) : 0.f;
        pre_b = (threadIdx.x < DELTA_GROUP && i0 + (int)threadIdx.x < n) ? bp[(size_t)(i0 + threadIdx.x) * p.ldb] : 0.f;
    };
    fetch(0);
    for (int i0 = 0; i0 < n; i0 += DELTA_GROUP) {
        __syncthreads();                       // the group before is no longer read
#pragma unroll
        for (int tt = 0; tt < DELTA_GROUP; tt++)
#pragma unroll
            for (int x = 0; x < RP; x++)
                if (threadIdx.x + x * DELTA_THREADS < DKP) {
#pragma unroll
                    for (int arr = 0; arr < 3; arr++) stage[tt * TOKEN + arr * DKP + place[x]] = pre[tt][arr][x];
                }
        if (vt < DELTA_GROUP) stage[vt * TOKEN + 3 * DKP + vc] = pre_v;
        if (threadIdx.x < DELTA_GROUP) stage[threadIdx.x * TOKEN + 3 * DKP + DELTA_COLS] = pre_b;
        __syncthreads();
        if (i0 + DELTA_GROUP < n) fetch(i0 + DELTA_GROUP);
        float op[DELTA_GROUP];                 // every token's share of o, summed over the column's lanes behind the group
#pragma unroll
        for (int tt = 0; tt < DELTA_GROUP; tt++) {
            const float* tk = stage + tt * TOKEN + part * 4;
            const float* tq = tk + DKP;
            const float* tg = tq + DKP;
            const float v = stage[tt * TOKEN + 3 * DKP + col], beta = stage[tt * TOKEN + 3 * DKP + DELTA_COLS];
            float k[RPT];
            float pr[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < RPT; j += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(tk + j * DELTA_TPC), g4 = *reinterpret_cast<const float4*>(tg + j * DELTA_TPC);
                k[j] = k4.x; k[j + 1] = k4.y; k[j + 2] = k4.z; k[j + 3] = k4.w;
                s[j] *= g4.x; s[j + 1] *= g4.y; s[j + 2] *= g4.z; s[j + 3] *= g4.w;
                pr[0] = fmaf(s[j], k4.x, pr[0]); pr[1] = fmaf(s[j + 1], k4.y, pr[1]);
                pr[2] = fmaf(s[j + 2], k4.z, pr[2]); pr[3] = fmaf(s[j + 3], k4.w, pr[3]);
            }
            const float pred = part_sum((pr[0] + pr[1]) + (pr[2] + pr[3]));
            const float u = beta * (v - pred);
            float ou[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < RPT; j += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(tq + j * DELTA_TPC);
                s[j] = fmaf(k[j], u, s[j]); s[j + 1] = fmaf(k[j + 1], u, s[j + 1]);
                s[j + 2] = fmaf(k[j + 2], u, s[j + 2]); s[j + 3] = fmaf(k[j + 3], u, s[j + 3]);
                ou[0] = fmaf(s[j], q4.x, ou[0]); ou[1] = fmaf(s[j + 1], q4.y, ou[1]);
                ou[2] = fmaf(s[j + 2], q4.z, ou[2]); ou[3] = fmaf(s[j + 3], q4.w, ou[3]);
            }
            op[tt] = (ou[0] + ou[1]) + (ou[2] + ou[3]);
        }
#pragma unroll
        for (int tt = 0; tt < DELTA_GROUP; tt++) {
            const float o = part_sum(op[tt]);
            if (live && part == 0 && i0 + tt < n) p.out[(size_t)(tok0 + i0 + tt) * hd + (size_t)h * p.dv + c] = o;
        }
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
    const int shares = tokens >= 512 ? 1 : (heads * dk >= 2048 ? 8 : (heads * dk >= 512 ? 2 : 1));   // few tokens: several blocks a token
    HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(delta_prep_kernel<T>, dim3(tokens, shares), dim3(128), 0, stream, p));
    return hymt2_check_launch("delta_prep");
}

HYMT2_API int hymt2_delta_scan_max_dk() { return 256; }

HYMT2_API int hymt2_delta_scan(float* out, const float* q, const float* k, const float* decay, const float* beta, long ldb, const void* v,
                               long ldv, int dtype, void* state, long state_offset, long state_stride, const int* cu_seqlens,
                               const int* slot_ids, const int* kv_lens, int batch, int max_new_tokens, int heads, int kv_heads, int dk,
                               int dv, cudaStream_t stream) {
    if (batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && heads > 0 && heads <= 65535 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0,
                  "delta_scan: bad sizes");
    HYMT2_REQUIRE(dk <= 256, "delta_scan: %d key channels a head; up to 256 are taken", dk);
    HYMT2_REQUIRE(state_offset % 4 == 0 && state_stride % 4 == 0, "delta_scan: the state must be 4-byte aligned");
    DeltaScanParams p;
    p.out = out; p.q = q; p.k = k; p.decay = decay; p.beta = beta; p.v = v; p.state = (uint8_t*)state + state_offset;
    p.state_stride = state_stride; p.ldv = ldv; p.ldb = ldb; p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.heads = heads; p.kv_heads = kv_heads; p.dk = dk; p.dv = dv;
#define DELTA_LAUNCH(RPT)                                                                                             \
    do {                                                                                                              \
        const dim3 grid((dv + DELTA_COLS - 1) / DELTA_COLS, heads, batch);                                            \
        if (max_new_tokens == 1)                                                                                      \
            HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(delta_scan_kernel<T, RPT, 1>, grid, dim3(DELTA_THREADS), 0, stream, p)); \
        else                                                                                                          \
            HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(delta_scan_kernel<T, RPT, 8>, grid, dim3(DELTA_THREADS), 0, stream, p)); \
    } while (0)
    if (dk <= 32) DELTA_LAUNCH(4);
    else if (dk <= 64) DELTA_LAUNCH(8);
    else if (dk <= 128) DELTA_LAUNCH(16);
    else DELTA_LAUNCH(32);
#undef DELTA_LAUNCH
    return hymt2_check_launch("delta_scan");
}
