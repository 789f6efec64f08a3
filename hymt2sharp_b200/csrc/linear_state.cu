// Mixers whose memory is a matrix per head instead of a list of keys: S [dk, dv] float32 per (sequence, head), carried from
// token to token and from step to step in the sequence's state row.
//
//   fixed decay    S = g_h S + (c k_t) v_t^T;                o_t = S^T q_t                    (g_h a constant of the head, c a constant)
//   token decay    o_t = (S + diag(u_h) k_t v_t^T)^T r_t;    S = diag(w_t) S + k_t v_t^T      (w_t = exp(-exp(x_t + w0)) per channel)
//
// Both forms are independent per value column j of S, so a block owns a tile of columns of one (sequence, head) and a thread
// one column: S[:, j] in registers where dk is one of the sizes compiled for (columns of 128 rows in two halves, on two threads
// whose sums meet in shared memory), in shared memory otherwise.  Everything that
// enters the recurrence is float32; q, k, v arrive in the engine's compute type.  The scan writes o as float32; the norm of
// each head's o, the gain and the gate follow in `head_norm_gate`.
//
// Long portions run in three passes over chunks of CHUNK tokens instead of one serial walk (the recurrences compose):
//   pass 1  per chunk, from a zero state: the chunk's own contribution B_c to the state, and the product A_c of its decays
//   pass 2  per (sequence, head): the state at every chunk's start, S_c = A_(c-1) S_(c-1) + B_(c-1), serial over chunks
//   pass 3  per chunk: the walk over its tokens from S_c, which writes o
// so a prompt of thousands of tokens keeps the whole device busy.  The order of the sums inside a chunk is the serial one; the
// state at a chunk's start is the same value in another association, which differs from the serial walk by rounding only.
//
// `token_shift`: the inputs of a time-mixing layer, m_s[t] = h[t] + (h[t-1] - h[t]) * mu_s for several s at once, with the last
// h of the step before taken from (and the step's last h written to) the state row.
#include "common.cuh"

namespace {

constexpr int CHUNK = 64;          // tokens of a chunk of the three-pass form
constexpr int MIN_CHUNKED = 192;   // a step whose longest portion has at least this many tokens runs in three passes

struct ScanParams {
    float* out;                    // [tokens][heads * dv] float32
    const void* q;                 // q (fixed decay) or r (token decay): rows of heads * dk
    const void* k;
    const void* v;                 // rows of heads * dv
    const float* x;                // token decay: [tokens][heads * dk] float32, the decay's inner exponent without w0
    const float* w0;               // token decay: [heads * dk]
    const float* u;                // token decay: [heads * dk] bonus
    const float* decay;            // fixed decay: [heads]
    float k_scale;                 // fixed decay: keys are multiplied by this
    long ldq, ldk, ldv, ldx;       // row strides in elements
    uint8_t* state;                // the cache's state rows
    long state_offset, state_stride;   // bytes
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    int heads, dk, dv;
    // the three-pass form
    float* chunk_B;                // [chunks][heads][dk][dv]
    float* chunk_A;                // token decay: [chunks][heads][dk] products of decays; fixed decay: unused
    const int* chunk_seq;          // [chunks] sequence of a chunk
    const int* chunk_first;        // [chunks] first token (row) of a chunk
    const int* chunk_len;          // [chunks]
    const int* seq_chunk0;         // [sequences + 1] first chunk of a sequence
};

// One thread's walk over `n` tokens for its column j of one head.  MODE 0: fixed decay, 1: token decay.
// WRITE_OUT: o is written; the state goes from S (in/out).  `vecs` is shared memory for two tokens' vectors, `us` for the
// bonus (token decay).  With DK > 0 (state in registers) the next token's vectors are loaded into registers in front of the
// current token's sums and stored to shared memory behind them, so that the loads' latency lies under the arithmetic; the
// vectors are read back four entries at a time, and o is summed in four partial sums over i mod 4, added as (0 + 1) + (2 + 3).
// SPLIT threads share a column: thread `part` holds rows part * DK / SPLIT onward, the parts' sums of o meet in `partial`
// (shared, [2][SPLIT][columns]) and part 0 adds them in ascending order behind the token's barrier.
template <typename T, int MODE, int DK, int SPLIT, bool WRITE_OUT>
__device__ __forceinline__ void walk(const ScanParams& p, int head, int j, bool live, int row0, int n, float* S, int sstride,
                                     float* vecs, const float* us, float gh, int part, int cols, float* partial) {
    const int dk = DK > 0 ? DK : p.dk;
    const int nvec = MODE == 0 ? 2 : 3;              // q, k (, w) per token
    const T* q = (const T*)p.q + (size_t)head * dk;
    const T* k = (const T*)p.k + (size_t)head * dk;
    const T* v = (const T*)p.v + (size_t)head * p.dv;
    const float* xx = MODE == 1 ? p.x + (size_t)head * dk : nullptr;
    const float* w0 = MODE == 1 ? p.w0 + (size_t)head * dk : nullptr;
    auto stage = [&](int t, float* dst) {
        const size_t r = (size_t)(row0 + t);
        for (int i = threadIdx.x; i < dk; i += blockDim.x) {
            dst[i] = to_float(q[r * p.ldq + i]);
            const float kk = to_float(k[r * p.ldk + i]);
            dst[dk + i] = MODE == 0 ? kk * p.k_scale : kk;
            if (MODE == 1) dst[2 * dk + i] = expf(-expf(xx[r * p.ldx + i] + w0[i]));
        }
    };
    stage(0, vecs);
    __syncthreads();
    if (DK > 0) {
        constexpr int PER = DK > 0 ? (DK + 31) / 32 : 1;   // entries of a vector that one thread fetches (blocks of 32 or more threads)
        float vnext = live ? to_float(v[(size_t)row0 * p.ldv + j]) : 0.f;
        for (int t = 0; t < n; t++) {
            const float* cur = vecs + (size_t)(t & 1) * nvec * dk;
            float* nxt = vecs + (size_t)((t + 1) & 1) * nvec * dk;
            const float vj = vnext;
            const bool more = t + 1 < n;
            T fq[PER], fk[PER];
            float fx[PER];
            if (more) {
                const size_t r = (size_t)(row0 + t + 1);
#pragma unroll
                for (int e = 0; e < PER; e++) {
                    const int i = threadIdx.x + e * blockDim.x;
                    if (i < dk) {
                        fq[e] = q[r * p.ldq + i];
                        fk[e] = k[r * p.ldk + i];
                        if (MODE == 1) fx[e] = xx[r * p.ldx + i];
                    }
                }
                if (live) vnext = to_float(v[r * p.ldv + j]);
            }
            constexpr int ROWS = (DK > 0 ? DK : 4) / SPLIT;
            const float4* cq = reinterpret_cast<const float4*>(cur) + part * (ROWS / 4);
            const float4* ck = reinterpret_cast<const float4*>(cur + dk) + part * (ROWS / 4);
            const float4* cw = reinterpret_cast<const float4*>(cur + 2 * dk) + part * (ROWS / 4);
            const float4* cu = reinterpret_cast<const float4*>(us) + part * (ROWS / 4);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int g = 0; g < ROWS / 4; g++) {
                const float4 q4 = cq[g], k4 = ck[g];
                float* s = S + 4 * g;
                if (MODE == 0) {
                    s[0] = fmaf(gh, s[0], k4.x * vj); a0 = fmaf(s[0], q4.x, a0);
                    s[1] = fmaf(gh, s[1], k4.y * vj); a1 = fmaf(s[1], q4.y, a1);
                    s[2] = fmaf(gh, s[2], k4.z * vj); a2 = fmaf(s[2], q4.z, a2);
                    s[3] = fmaf(gh, s[3], k4.w * vj); a3 = fmaf(s[3], q4.w, a3);
                } else {
                    const float4 w4 = cw[g], u4 = cu[g];
                    const float kx = k4.x * vj, ky = k4.y * vj, kz = k4.z * vj, kw = k4.w * vj;
                    a0 = fmaf(q4.x, fmaf(u4.x, kx, s[0]), a0); s[0] = fmaf(w4.x, s[0], kx);
                    a1 = fmaf(q4.y, fmaf(u4.y, ky, s[1]), a1); s[1] = fmaf(w4.y, s[1], ky);
                    a2 = fmaf(q4.z, fmaf(u4.z, kz, s[2]), a2); s[2] = fmaf(w4.z, s[2], kz);
                    a3 = fmaf(q4.w, fmaf(u4.w, kw, s[3]), a3); s[3] = fmaf(w4.w, s[3], kw);
                }
            }
            if (more) {
#pragma unroll
                for (int e = 0; e < PER; e++) {
                    const int i = threadIdx.x + e * blockDim.x;
                    if (i < dk) {
                        nxt[i] = to_float(fq[e]);
                        const float kk = to_float(fk[e]);
                        nxt[dk + i] = MODE == 0 ? kk * p.k_scale : kk;
                        if (MODE == 1) nxt[2 * dk + i] = expf(-expf(fx[e] + w0[i]));
                    }
                }
            }
            const float mine = (a0 + a1) + (a2 + a3);
            if constexpr (SPLIT == 1) {
                if (WRITE_OUT && live) p.out[(size_t)(row0 + t) * p.heads * p.dv + (size_t)head * p.dv + j] = mine;
                __syncthreads();
            } else {
                float* meet = partial + (size_t)(t & 1) * SPLIT * cols;
                const int col = threadIdx.x - part * cols;
                if (WRITE_OUT) meet[part * cols + col] = mine;
                __syncthreads();
                if (WRITE_OUT && live && part == 0) {
                    float o = meet[col];
#pragma unroll
                    for (int r = 1; r < SPLIT; r++) o += meet[r * cols + col];
                    p.out[(size_t)(row0 + t) * p.heads * p.dv + (size_t)head * p.dv + j] = o;
                }
            }
        }
        return;
    }
    for (int t = 0; t < n; t++) {
        float* cur = vecs + (size_t)(t & 1) * nvec * dk;
        if (t + 1 < n) stage(t + 1, vecs + (size_t)((t + 1) & 1) * nvec * dk);
        const float vj = live ? to_float(v[(size_t)(row0 + t) * p.ldv + j]) : 0.f;
        float acc = 0.f;
        for (int i = 0; i < dk; i++) {
            float s = S[(size_t)i * sstride];
            if (MODE == 0) {
                s = fmaf(gh, s, cur[dk + i] * vj);
                acc = fmaf(s, cur[i], acc);
            } else {
                const float kv = cur[dk + i] * vj;
                acc = fmaf(cur[i], fmaf(us[i], kv, s), acc);
                s = fmaf(cur[2 * dk + i], s, kv);
            }
            S[(size_t)i * sstride] = s;
        }
        if (WRITE_OUT && live) p.out[(size_t)(row0 + t) * p.heads * p.dv + (size_t)head * p.dv + j] = acc;
        __syncthreads();
    }
}

// Pass 1 with the state in registers: a chunk's contribution to the state from zero has no token-by-token dependency,
//     B[i][j] = sum_t c_t[i] v_t[j],   c_t[i] = k_t[i] * (the product of the decays of the tokens behind t in the chunk)[i],
// so groups of GATHER_TOKENS tokens are staged at once (all their loads in flight together), from the chunk's last group to
// its first, with the product of the decays carried from group to group: fixed decay, a scalar; token decay, a register per
// key entry that a thread owns, which at the end is the chunk's whole product (returned through `A` when given).  One fused
// multiply-add an entry and token.  `kp` and `wv` are shared memory of GATHER_TOKENS * dk floats each (fixed decay: `wv`
// holds the decay's first GATHER_TOKENS powers).
constexpr int GATHER_TOKENS = 8;

template <typename T, int MODE, int DK, int SPLIT>
__device__ __forceinline__ void gather(const ScanParams& p, int head, int j, bool live, int row0, int n, float* S, float* kp, float* wv,
                                       float gh, int part, float* A) {
    constexpr int TB = GATHER_TOKENS, ROWS = DK / SPLIT;
    constexpr int OWN = (DK + 31) / 32;               // key entries that one thread owns (blocks of 32 or more threads)
    const T* k = (const T*)p.k + (size_t)head * DK;
    const T* v = (const T*)p.v + (size_t)head * p.dv;
    const float* xx = MODE == 1 ? p.x + (size_t)head * DK : nullptr;
    const float* w0 = MODE == 1 ? p.w0 + (size_t)head * DK : nullptr;
    float behind = 1.f;                               // fixed decay: the decay to the power of the tokens behind the group
    float run[OWN];                                   // token decay: the product of the decays behind the group, per owned entry
#pragma unroll
    for (int e = 0; e < OWN; e++) run[e] = 1.f;
    if (MODE == 0) {                                  // fixed decay: wv[d] = decay^d for the tokens behind one inside its group
        if (threadIdx.x < TB) {
            float f = 1.f;
            for (int b = 0; b < (int)threadIdx.x; b++) f *= gh;
            wv[threadIdx.x] = f;
        }
        __syncthreads();
    }
    for (int g1 = n; g1 > 0; g1 -= TB) {
        const int g0 = g1 > TB ? g1 - TB : 0, len = g1 - g0;
        const float scale_behind = p.k_scale * behind;
        float vv[TB];
#pragma unroll
        for (int tt = 0; tt < TB; tt++) vv[tt] = (live && tt < len) ? to_float(v[(size_t)(row0 + g0 + tt) * p.ldv + j]) : 0.f;
        // FLIGHT loads of a thread are issued together in front of their use
        constexpr int FLIGHT = 8;
        for (int base = threadIdx.x; base < len * DK; base += FLIGHT * blockDim.x) {
            T kr[FLIGHT];
            float xr[FLIGHT];
#pragma unroll
            for (int m = 0; m < FLIGHT; m++) {
                const int e = base + m * blockDim.x;
                if (e < len * DK) {
                    const int tt = e / DK, i = e - tt * DK;
                    const size_t r = (size_t)(row0 + g0 + tt);
                    kr[m] = k[r * p.ldk + i];
                    if (MODE == 1) xr[m] = xx[r * p.ldx + i];
                }
            }
#pragma unroll
            for (int m = 0; m < FLIGHT; m++) {
                const int e = base + m * blockDim.x;
                if (e < len * DK) {
                    const int tt = e / DK, i = e - tt * DK;
                    if (MODE == 0) {
                        kp[e] = to_float(kr[m]) * (scale_behind * wv[len - 1 - tt]);
                    } else {
                        kp[e] = to_float(kr[m]);
                        wv[e] = expf(-expf(xr[m] + w0[i]));
                    }
                }
            }
        }
        __syncthreads();
        if (MODE == 0) {
            for (int b = 0; b < len; b++) behind *= gh;
        } else {
#pragma unroll
            for (int e = 0; e < OWN; e++) {
                const int i = threadIdx.x + e * blockDim.x;
                if (i < DK) {
                    float w = run[e];
                    for (int tt = len - 1; tt >= 0; tt--) {
                        kp[tt * DK + i] *= w;
                        w *= wv[tt * DK + i];
                    }
                    run[e] = w;
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int tt = 0; tt < TB; tt++) {
            if (tt < len) {
                const float4* c4 = reinterpret_cast<const float4*>(kp + tt * DK) + part * (ROWS / 4);
                const float vj = vv[tt];
#pragma unroll
                for (int g = 0; g < ROWS / 4; g++) {
                    const float4 c = c4[g];
                    float* s = S + 4 * g;
                    s[0] = fmaf(c.x, vj, s[0]);
                    s[1] = fmaf(c.y, vj, s[1]);
                    s[2] = fmaf(c.z, vj, s[2]);
                    s[3] = fmaf(c.w, vj, s[3]);
                }
            }
        }
        __syncthreads();                              // the next group overwrites kp
    }
    if (MODE == 1 && A) {
#pragma unroll
        for (int e = 0; e < OWN; e++) {
            const int i = threadIdx.x + e * blockDim.x;
            if (i < DK) A[i] = run[e];
        }
    }
}

// PASS 0: the serial form, grid (column tiles, heads, sequences).  PASS 1 and 3: grid (column tiles, heads, chunks).
template <typename T, int MODE, int DK, int PASS>
__global__ void __launch_bounds__(128)
scan_kernel(ScanParams p) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int dk = DK > 0 ? DK : p.dk;
    const int nvec = MODE == 0 ? 2 : 3;
    float* vecs = smem;                                   // [2][nvec][dk]
    float* us = smem + 2 * nvec * dk;                     // [dk] the bonus (token decay)
    constexpr int SPLIT = DK == 128 ? 2 : 1;              // threads that share a column (each holds DK / SPLIT rows of it)
    float* partial = us + (MODE == 1 ? dk : 0);           // [2][SPLIT][columns] when SPLIT > 1
    float* shared_state = partial;                        // [dk][blockDim.x] when DK == 0
    if (MODE == 1 && !(PASS == 1 && DK > 0))              // (pass 1 with the state in registers lays the shared memory out anew)
        for (int i = threadIdx.x; i < dk; i += blockDim.x) us[i] = p.u[(size_t)blockIdx.y * dk + i];   // (visible behind the walk's first barrier)
    const int head = blockIdx.y;
    const int cols = blockDim.x / SPLIT;
    const int part = threadIdx.x / cols;
    const int j = blockIdx.x * cols + (threadIdx.x - part * cols);
    const bool live = j < p.dv;
    int seq, row0, n, chunk = 0;
    bool from_zero, keep;
    if (PASS == 0) {
        seq = blockIdx.z;
        row0 = p.cu_seqlens[seq];
        n = p.cu_seqlens[seq + 1] - row0;
        from_zero = p.kv_lens[seq] - n == 0;
        keep = true;
    } else {
        chunk = blockIdx.z;
        seq = p.chunk_seq[chunk];
        row0 = p.chunk_first[chunk];
        n = p.chunk_len[chunk];
        from_zero = PASS == 1;
        keep = false;
    }
    if (n <= 0) return;
    const int slot = p.slot_ids[seq];
    if (slot < 0) {                                       // a padding row: zeros out, nothing remembered
        if (PASS != 1 && live && part == 0)
            for (int t = 0; t < n; t++) p.out[(size_t)(row0 + t) * p.heads * p.dv + (size_t)head * p.dv + j] = 0.f;
        return;
    }
    float* st = reinterpret_cast<float*>(p.state + (size_t)slot * p.state_stride + p.state_offset) + (size_t)head * dk * p.dv;
    const float* from = PASS == 3 ? p.chunk_B + ((size_t)chunk * p.heads + head) * dk * p.dv : st;   // pass 2 left S_c in chunk_B
    constexpr int ROWS = DK > 0 ? DK / SPLIT : 1;         // rows of the column that this thread holds (DK == 0: all dk, in shared memory)
    const int rows = DK > 0 ? ROWS : dk, i0 = part * ROWS;
    float reg[ROWS];
    float* S = DK > 0 ? reg : shared_state + threadIdx.x;
    const int sstride = DK > 0 ? 1 : blockDim.x;
    if (DK > 0) {
#pragma unroll
        for (int i = 0; i < ROWS; i++) reg[i] = (!from_zero && live) ? from[(size_t)(i0 + i) * p.dv + j] : 0.f;
    } else {
        for (int i = 0; i < dk; i++) S[(size_t)i * sstride] = (!from_zero && live) ? from[(size_t)i * p.dv + j] : 0.f;
    }
    const float gh = MODE == 0 ? p.decay[head] : 0.f;
    if constexpr (PASS == 1 && DK > 0) {
        float* A = (MODE == 1 && blockIdx.x == 0) ? p.chunk_A + ((size_t)chunk * p.heads + head) * dk : nullptr;
        gather<T, MODE, DK, SPLIT>(p, head, j, live, row0, n, S, smem, smem + GATHER_TOKENS * DK, gh, part, A);
    } else if (PASS == 1) {
        walk<T, MODE, DK, SPLIT, false>(p, head, j, live, row0, n, S, sstride, vecs, us, gh, part, cols, partial);
    } else {
        walk<T, MODE, DK, SPLIT, true>(p, head, j, live, row0, n, S, sstride, vecs, us, gh, part, cols, partial);
    }
    if (PASS == 1) {
        float* B = p.chunk_B + ((size_t)chunk * p.heads + head) * dk * p.dv;
        if (live) {
            if (DK > 0) {
#pragma unroll
                for (int i = 0; i < ROWS; i++) B[(size_t)(i0 + i) * p.dv + j] = reg[i];
            } else {
                for (int i = 0; i < rows; i++) B[(size_t)i * p.dv + j] = S[(size_t)i * sstride];
            }
        }
        if (MODE == 1 && DK == 0 && blockIdx.x == 0) {    // the product of the chunk's decays per channel (DK > 0: made above)
            float* A = p.chunk_A + ((size_t)chunk * p.heads + head) * dk;
            for (int i = threadIdx.x; i < dk; i += blockDim.x) {
                float a = 1.f;
                for (int t = 0; t < n; t++)
                    a *= expf(-expf(p.x[(size_t)(row0 + t) * p.ldx + (size_t)head * dk + i] + p.w0[(size_t)head * dk + i]));
                A[i] = a;
            }
        }
    } else if (keep && live) {
        if (DK > 0) {
#pragma unroll
            for (int i = 0; i < ROWS; i++) st[(size_t)(i0 + i) * p.dv + j] = reg[i];
        } else {
            for (int i = 0; i < rows; i++) st[(size_t)i * p.dv + j] = S[(size_t)i * sstride];
        }
    }
}

// Pass 2: S at every chunk's start.  A thread owns one entry (i, j) of one (sequence, head) and walks the sequence's chunks:
// chunk_B[c] holds B_c on entry and S_c (the state in FRONT of chunk c) on exit; the state row receives the state behind the
// last chunk.
template <int MODE>
__global__ void __launch_bounds__(256)
scan_carry_kernel(ScanParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.z, head = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int per = p.dk * p.dv;
    if (e >= per) return;
    const int slot = p.slot_ids[seq];
    const int c0 = p.seq_chunk0[seq], c1 = p.seq_chunk0[seq + 1];
    if (slot < 0 || c1 <= c0) return;
    const int n = p.cu_seqlens[seq + 1] - p.cu_seqlens[seq];
    float* st = reinterpret_cast<float*>(p.state + (size_t)slot * p.state_stride + p.state_offset) + (size_t)head * per;
    float s = p.kv_lens[seq] - n == 0 ? 0.f : st[e];
    const int i = e / p.dv;
    const float gh = MODE == 0 ? p.decay[head] : 0.f;
    // fixed decay: a chunk's factor is the decay multiplied up over its tokens; all chunks but a sequence's last have the first
    // one's length, so that product is made once.  The loads of AHEAD chunks are issued together in front of their serial sums.
    constexpr int AHEAD = 4;
    const int len0 = p.chunk_len[c0];
    float a_first = 1.f;
    if (MODE == 0)
        for (int t = 0; t < len0; t++) a_first *= gh;
    for (int c = c0; c < c1; c += AHEAD) {
        float a[AHEAD], b[AHEAD];
#pragma unroll
        for (int r = 0; r < AHEAD; r++) {
            if (c + r >= c1) continue;
            b[r] = p.chunk_B[((size_t)(c + r) * p.heads + head) * per + e];
            if (MODE == 0) {
                const int len = p.chunk_len[c + r];
                a[r] = a_first;
                if (len != len0) {
                    a[r] = 1.f;
                    for (int t = 0; t < len; t++) a[r] *= gh;
                }
            } else {
                a[r] = p.chunk_A[((size_t)(c + r) * p.heads + head) * p.dk + i];
            }
        }
#pragma unroll
        for (int r = 0; r < AHEAD; r++) {
            if (c + r >= c1) continue;
            p.chunk_B[((size_t)(c + r) * p.heads + head) * per + e] = s;
            s = fmaf(a[r], s, b[r]);
        }
    }
    st[e] = s;
}

// out[t, head, :] = o[t, head, :] / sqrt(mean(o^2) + eps) * (weight[head, :] if given) * act(gate[t, head, :]), a warp per
// (token, head); act: 0 none (no gate), 1 silu.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ gate, long ldg, const float* __restrict__ weight,
                      long items, int heads, int dv, float eps, int gate_sigmoid) {
    pdl_wait();
    pdl_launch_dependents();
    const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= items) return;
    const long t = item / heads;
    const int head = (int)(item % heads);
    const float* row = o + (size_t)item * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        float y = row[c] * r;
        if (weight) y *= weight[(size_t)head * dv + c];
        if (gate) {
            const float g = to_float(gate[(size_t)t * ldg + (size_t)head * dv + c]);
            y *= (gate_sigmoid ? 1.0f : g) / (1.0f + expf(-g));
        }
        out[(size_t)item * dv + c] = from_float<T>(y);
    }
}

// The same with a head's entries in registers: lane l holds entries [128 p + 4 l, 128 p + 4 l + 4) for p < P, read once in
// 16-byte accesses; the gate and the output move four entries an access.
template <typename T, int P>
__global__ void __launch_bounds__(128)
head_norm_gate_wide_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ gate, long ldg,
                           const float* __restrict__ weight, long items, int heads, int dv, float eps, int gate_sigmoid) {
    pdl_wait();
    pdl_launch_dependents();
    const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= items) return;
    const long t = item / heads;
    const int head = (int)(item % heads);
    const float* row = o + (size_t)item * dv;
    Pack<float, 4> x[P];
    Pack<T, 4> g[P];
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int c = p * 128 + lane * 4;
        if (c < dv) {
            x[p] = load_pack<float, 4>(row + c);
            if (gate) g[p] = load_pack<T, 4>(gate + (size_t)t * ldg + (size_t)head * dv + c);
#pragma unroll
            for (int e = 0; e < 4; e++) ss = fmaf(x[p].v[e], x[p].v[e], ss);
        }
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int c = p * 128 + lane * 4;
        if (c < dv) {
            Pack<float, 4> w;
            if (weight) w = load_pack<float, 4>(weight + (size_t)head * dv + c);
            Pack<T, 4> y;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = x[p].v[e] * r;
                if (weight) v *= w.v[e];
                if (gate) {
                    const float gv = to_float(g[p].v[e]);
                    v *= (gate_sigmoid ? 1.0f : gv) / (1.0f + expf(-gv));
                }
                y.v[e] = from_float<T>(v);
            }
            store_pack<T, 4>(out + (size_t)item * dv + c, y);
        }
    }
}

// mixes[t][s * width + c] = h[t][c] + (h[t-1][c] - h[t][c]) * mu[s][c]; a sequence's first new token takes h[t-1] from the state
// row (zeros at position 0), and the thread of that token also writes the step's last h there: one thread reads and renews.
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(T* __restrict__ mixes, const T* __restrict__ h, long ldh, const float* __restrict__ mu, int count, uint8_t* state,
                   long state_offset, long state_stride, const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ slot_ids, const int* __restrict__ kv_lens, int tokens, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)tokens * width) return;
    const int t = (int)(idx / width), c = (int)(idx % width);
    const int seq = token_seq[t];
    const int first = cu_seqlens[seq], last = cu_seqlens[seq + 1] - 1;
    const float cur = to_float(h[(size_t)t * ldh + c]);
    float prev;
    if (t > first) {
        prev = to_float(h[(size_t)(t - 1) * ldh + c]);
    } else {
        const int slot = slot_ids[seq];
        prev = 0.f;
        if (slot >= 0) {
            float* st = reinterpret_cast<float*>(state + (size_t)slot * state_stride + state_offset);
            const bool at_start = kv_lens[seq] - (last - first + 1) == 0;
            if (!at_start) prev = st[c];
            st[c] = to_float(h[(size_t)last * ldh + c]);
        }
    }
    for (int s = 0; s < count; s++)
        mixes[(size_t)t * count * width + (size_t)s * width + c] = from_float<T>(fmaf(prev - cur, mu[(size_t)s * width + c], cur));
}

template <typename T, int MODE, int DK, int PASS>
int launch_scan(const ScanParams& p, int threads, int z, cudaStream_t stream) {
    const int cols = DK == 128 ? threads / 2 : threads;   // (the kernel's SPLIT)
    const int tiles = (p.dv + cols - 1) / cols;
    const int dk = p.dk, nvec = MODE == 0 ? 2 : 3;
    size_t smem = ((size_t)2 * nvec * dk + (MODE == 1 ? dk : 0) + (DK > 0 ? (size_t)2 * threads : (size_t)dk * threads)) * sizeof(float);
    if (PASS == 1 && DK > 0) smem = (size_t)2 * GATHER_TOKENS * DK * sizeof(float);   // the staged groups (fixed decay: its powers)
    if (smem > 48 * 1024) {
        HYMT2_REQUIRE(smem <= 200 * 1024, "linear_scan: heads of %d key entries are too large", dk);
        cudaFuncSetAttribute(scan_kernel<T, MODE, DK, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    launch_pdl(scan_kernel<T, MODE, DK, PASS>, dim3(tiles, p.heads, z), dim3(threads), smem, stream, p);
    return HYMT2_OK;
}

template <typename T, int MODE, int PASS>
int launch_scan_dk(const ScanParams& p, int z, cudaStream_t stream) {
    // columns a block: enough blocks to fill the device matter more than wide blocks
    const int threads = p.dv >= 64 ? 64 : 32;
    switch (p.dk) {
        case 16: return launch_scan<T, MODE, 16, PASS>(p, threads, z, stream);
        case 32: return launch_scan<T, MODE, 32, PASS>(p, threads, z, stream);
        case 64: return launch_scan<T, MODE, 64, PASS>(p, threads, z, stream);
        case 128: return launch_scan<T, MODE, 128, PASS>(p, p.dv > 16 ? 64 : 32, z, stream);   // two threads a column: 32 or 16 columns a block
        default: return launch_scan<T, MODE, 0, PASS>(p, threads, z, stream);
    }
}

}  // namespace

// Floats and ints of scratch that the three-pass form needs for a step of `chunks` chunks (0: the step runs serially).
HYMT2_API int hymt2_linear_scan_chunk() { return CHUNK; }
HYMT2_API int hymt2_linear_scan_min_chunked() { return MIN_CHUNKED; }

// mode 0: fixed decay per head (decay [heads], k_scale); mode 1: decay per token and channel with a bonus (x, w0, u).
// chunks > 0: the three-pass form over the chunks that the host laid out (chunk_* and seq_chunk0 int32 on the device, chunk_B
// [chunks * heads * dk * dv] and chunk_A [chunks * heads * dk] float32 scratch).
HYMT2_API int hymt2_linear_scan(float* out, const void* q, const void* k, const void* v, int dtype, long ldq, long ldk, long ldv,
                                const float* x, long ldx, const float* w0, const float* u, const float* decay, float k_scale, int mode,
                                uint8_t* state, long state_offset, long state_stride, const int* cu_seqlens, const int* slot_ids,
                                const int* kv_lens, int batch, int heads, int dk, int dv, int chunks, float* chunk_B, float* chunk_A,
                                const int* chunk_seq, const int* chunk_first, const int* chunk_len, const int* seq_chunk0,
                                cudaStream_t stream) {
    if (batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && heads > 0 && dk > 0 && dv > 0, "linear_scan: bad sizes");
    HYMT2_REQUIRE(mode == 0 || mode == 1, "linear_scan: unknown mode %d", mode);
    HYMT2_REQUIRE(mode == 0 ? decay != nullptr : (x && w0 && u), "linear_scan: the decay's tensors are missing");
    HYMT2_REQUIRE(chunks == 0 || (chunk_B && chunk_seq && chunk_first && chunk_len && seq_chunk0 && (mode == 0 || chunk_A)),
                  "linear_scan: the chunked form needs its scratch");
    ScanParams p{out, q, k, v, x, w0, u, decay, k_scale, ldq, ldk, ldv, ldx, state, state_offset, state_stride, cu_seqlens, slot_ids,
                 kv_lens, heads, dk, dv, chunk_B, chunk_A, chunk_seq, chunk_first, chunk_len, seq_chunk0};
    int rc = HYMT2_OK;
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        if (chunks == 0) {
            rc = mode == 0 ? launch_scan_dk<T, 0, 0>(p, batch, stream) : launch_scan_dk<T, 1, 0>(p, batch, stream);
        } else {
            rc = mode == 0 ? launch_scan_dk<T, 0, 1>(p, chunks, stream) : launch_scan_dk<T, 1, 1>(p, chunks, stream);
            if (rc == HYMT2_OK) {
                const int per = dk * dv;
                if (mode == 0) launch_pdl(scan_carry_kernel<0>, dim3((per + 255) / 256, heads, batch), dim3(256), 0, stream, p);
                else launch_pdl(scan_carry_kernel<1>, dim3((per + 255) / 256, heads, batch), dim3(256), 0, stream, p);
                rc = mode == 0 ? launch_scan_dk<T, 0, 3>(p, chunks, stream) : launch_scan_dk<T, 1, 3>(p, chunks, stream);
            }
        }
    });
    if (rc != HYMT2_OK) return rc;
    return hymt2_check_launch("linear_scan");
}

HYMT2_API int hymt2_head_norm_gate(void* out, const float* o, const void* gate, long ldg, int dtype, const float* weight, int tokens,
                                   int heads, int dv, float eps, int gate_sigmoid, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && heads > 0 && dv > 0, "head_norm_gate: bad sizes");
    const long items = (long)tokens * heads;
    const dim3 grid((unsigned)((items + 3) / 4));
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        // a head in registers, four entries an access: widths that are multiples of 4 up to 512, every row start aligned
        const bool wide = dv % 4 == 0 && dv <= 512 && (uintptr_t)o % 16 == 0 && (uintptr_t)out % (4 * sizeof(T)) == 0 &&
                          (!gate || ((uintptr_t)gate % (4 * sizeof(T)) == 0 && ldg % 4 == 0)) && (!weight || (uintptr_t)weight % 16 == 0);
        if (wide && dv <= 128)
            launch_pdl(head_norm_gate_wide_kernel<T, 1>, grid, dim3(128), 0, stream, (T*)out, o, (const T*)gate, ldg, weight, items, heads, dv, eps, gate_sigmoid);
        else if (wide && dv <= 256)
            launch_pdl(head_norm_gate_wide_kernel<T, 2>, grid, dim3(128), 0, stream, (T*)out, o, (const T*)gate, ldg, weight, items, heads, dv, eps, gate_sigmoid);
        else if (wide)
            launch_pdl(head_norm_gate_wide_kernel<T, 4>, grid, dim3(128), 0, stream, (T*)out, o, (const T*)gate, ldg, weight, items, heads, dv, eps, gate_sigmoid);
        else
            launch_pdl(head_norm_gate_kernel<T>, grid, dim3(128), 0, stream, (T*)out, o, (const T*)gate, ldg, weight, items, heads, dv, eps, gate_sigmoid);
    });
    return hymt2_check_launch("head_norm_gate");
}

HYMT2_API int hymt2_token_shift(void* mixes, const void* h, long ldh, int dtype, const float* mu, int count, uint8_t* state,
                                long state_offset, long state_stride, const int* token_seq, const int* cu_seqlens, const int* slot_ids,
                                const int* kv_lens, int tokens, int width, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && width > 0 && count > 0, "token_shift: bad sizes");
    const long items = (long)tokens * width;
    HYMT2_DISPATCH_DTYPE(dtype, T, (launch_pdl(token_shift_kernel<T>, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, stream, (T*)mixes,
                                               (const T*)h, ldh, mu, count, state, state_offset, state_stride, token_seq, cu_seqlens,
                                               slot_ids, kv_lens, tokens, width)));
    return hymt2_check_launch("token_shift");
}
