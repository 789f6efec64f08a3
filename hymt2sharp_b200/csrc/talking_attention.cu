// Softmax attention whose heads talk to each other: the scores of all heads at a (query, key) pair are mixed by a stored matrix
// before the softmax,
//
//     raw_g(i, j) = (q_g(i) . k_g(j)) * scale * temp[g];     s_h(i, j) = sum_g talk[h, g] * raw_g(i, j)
//     p_h(i, j)   = exp(s_h(i, j)) / (exp(sink_h) + sum_j' exp(s_h(i, j')))        over the keys j' that i sees
//     out_h(i)    = sum_j p_h(i, j) v_h(j)        [* sigmoid(gate_h(i)), entry by entry, where a gate is given]
//
// so one block has to hold the scores of ALL heads for its tile of (queries x keys); everything else follows from that.  The
// sink is one more term of the denominator without a key or a value (a row starts from the running maximum sink_h and the
// running sum 1).  Which keys a query sees: j <= i, and with mask_kind CHUNK only those of its own chunk of `mask_size`
// positions (chunks counted from position 0 of the sequence), with mask_kind WINDOW only the last `mask_size`.
// Keys and values come from the paged cache (values may be another tensor than keys: here the keys before their rotation),
// query head h reads key/value head h / (heads / kv_heads).  Scores, softmax and sums are float32.
//
// `talk_prep` is what comes between the projections and this kernel: it rotates the first rot_dims entries of every q and k head
// in neighbouring pairs (2i, 2i+1) by position * inv_freq[i], writes q to its own tensor, the rotated k to the key plane and the
// UNROTATED k to the value plane of the token's cache row.
#include "common.cuh"

namespace {

enum { MASK_NONE = 0, MASK_CHUNK = 1, MASK_WINDOW = 2 };

struct TalkPrepParams {
    const void* x;        // [T, ldx]: q of all heads, then k of all key heads
    void* q_out;          // [T, heads * d]
    void* k_cache;        // plane bases
    void* v_cache;
    const int* block_table;
    const int* token_seq;
    const int* token_pos;
    const int* slot_ids;
    const float* inv_freq;
    long ldx;
    int table_stride, block_tokens, heads, kv_heads, d, rot_dims;
};

template <typename T>
__global__ void __launch_bounds__(128)
talk_prep_kernel(TalkPrepParams p) {
    extern __shared__ float cs[];   // [rot_dims / 2][2]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = p.token_pos[t];
    const int slot = p.slot_ids[p.token_seq[t]];
    const int half = p.rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, c;
        sincosf((float)pos * p.inv_freq[i], &sn, &c);
        cs[2 * i] = c;
        cs[2 * i + 1] = sn;
    }
    __syncthreads();
    const T* row = (const T*)p.x + (size_t)t * p.ldx;
    const int d = p.d, per = half + (d - p.rot_dims);      // work items of a head: pairs, then the entries that pass unchanged
    T* qo = (T*)p.q_out + (size_t)t * p.heads * d;
    for (int item = threadIdx.x; item < p.heads * per; item += blockDim.x) {
        const int h = item / per, i = item - h * per;
        const T* src = row + (size_t)h * d;
        T* dst = qo + (size_t)h * d;
        if (i < half) {
            const float a = to_float(src[2 * i]), b = to_float(src[2 * i + 1]);
            dst[2 * i] = from_float<T>(a * cs[2 * i] - b * cs[2 * i + 1]);
            dst[2 * i + 1] = from_float<T>(b * cs[2 * i] + a * cs[2 * i + 1]);
        } else {
            const int e = p.rot_dims + (i - half);
            dst[e] = src[e];
        }
    }
    if (slot < 0 || p.k_cache == nullptr) return;
    const int block = p.block_table[(size_t)slot * p.table_stride + pos / p.block_tokens];
    const size_t row0 = (size_t)block * p.kv_heads * p.block_tokens + (pos % p.block_tokens);
    const T* ksrc = row + (size_t)p.heads * d;
    for (int item = threadIdx.x; item < p.kv_heads * per; item += blockDim.x) {
        const int g = item / per, i = item - g * per;
        const T* src = ksrc + (size_t)g * d;
        T* kd = (T*)p.k_cache + (row0 + (size_t)g * p.block_tokens) * d;
        T* vd = (T*)p.v_cache + (row0 + (size_t)g * p.block_tokens) * d;
        if (i < half) {
            const T a0 = src[2 * i], b0 = src[2 * i + 1];
            const float a = to_float(a0), b = to_float(b0);
            kd[2 * i] = from_float<T>(a * cs[2 * i] - b * cs[2 * i + 1]);
            kd[2 * i + 1] = from_float<T>(b * cs[2 * i] + a * cs[2 * i + 1]);
            vd[2 * i] = a0;
            vd[2 * i + 1] = b0;
        } else {
            const int e = p.rot_dims + (i - half);
            kd[e] = src[e];
            vd[e] = src[e];
        }
    }
}

struct TalkParams {
    void* out;             // [T, heads * d]
    const void* q;         // [T, heads * d]
    const void* gate;      // [T, ldg] or null: the output is multiplied by its sigmoid entry by entry
    const void* k_cache;
    const void* v_cache;
    const int* block_table;
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    const float* talk;     // [heads, heads]
    const float* temp;     // [heads]
    const float* sink;     // [heads] or null
    long ldg;
    int table_stride, block_tokens, heads, kv_heads, d, mask_kind, mask_size, bk;
    float scale;
    // decode steps whose queries may see many keys: split s of a sequence takes the key tiles [s * split_keys, (s + 1) * split_keys)
    // behind the first tile that the query sees, and leaves its unnormalised sums (no sink, no gate) for `talk_merge`
    int split_keys, max_splits;
    float* part_o;         // [sequences, max_splits, heads * d]
    float* part_ml;        // [sequences, max_splits, 2 * heads]: running maximum, running sum
};

constexpr int TALK_THREADS = 256;

// the lowest position that the query at `pos` sees
__device__ __forceinline__ int lowest_seen(int pos, int kind, int size) {
    if (kind == MASK_CHUNK) return pos / size * size;
    if (kind == MASK_WINDOW) return max(0, pos - size + 1);
    return 0;
}

// BQ queries of one sequence against tiles of bk keys (bk <= 32, a divisor of block_tokens).  VEC: entries of a cache row
// that move in one access (d is a multiple of it).
template <typename T, int BQ, int VEC>
__global__ void __launch_bounds__(TALK_THREADS)
talking_attention_kernel(TalkParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.y;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    const bool split = p.split_keys > 0;                // (then BQ is 1 and blockIdx.x names the split)
    const int q0 = split ? 0 : blockIdx.x * BQ;
    if (q0 >= n) return;
    const int nq = min(BQ, n - q0);
    const int slot = p.slot_ids[b];
    const int H = p.heads, G = p.kv_heads, d = p.d, bk = p.bk, rep = H / G;
    const int hd = H * d;
    T* out = (T*)p.out + (size_t)(tok0 + q0) * hd;
    float* my_o = split ? p.part_o + ((size_t)b * p.max_splits + blockIdx.x) * hd : nullptr;
    float* my_ml = split ? p.part_ml + ((size_t)b * p.max_splits + blockIdx.x) * 2 * H : nullptr;
    if (slot < 0) {   // a padding row: a defined output, nothing read
        if (!split)
            for (int i = threadIdx.x; i < nq * hd; i += TALK_THREADS) out[i] = from_float<T>(0.f);
        else
            for (int i = threadIdx.x; i < H; i += TALK_THREADS) { my_ml[i] = -INFINITY; my_ml[H + i] = 0.f; }
        return;
    }
    const int start = p.kv_lens[b] - n;                 // position of the sequence's first new token
    const int pos_first = start + q0, pos_last = start + q0 + nq - 1;
    const int row_k = G * d + VEC;                      // a tile row of keys, padded by one access
    // shared memory, in this order: mix [H*H], sink [H], m/l/alpha [3*BQ*H], Q [BQ*H*d], O [BQ*H*d], raw and mixed scores
    // [2*BQ*H*bk] (float); then the key tile and the value tile [bk * row_k] of T
    float* mix = (float*)smem_raw;
    float* sinkv = mix + H * H;
    float* run_m = sinkv + H;
    float* run_l = run_m + BQ * H;
    float* alpha = run_l + BQ * H;
    float* Q = alpha + BQ * H;
    Q = (float*)(((uintptr_t)Q + 15) & ~(uintptr_t)15);
    float* O = Q + (size_t)BQ * hd;
    float* s_raw = O + (size_t)BQ * hd;
    float* s_mix = s_raw + (size_t)BQ * H * bk;
    T* Kt = (T*)(s_mix + (size_t)BQ * H * bk);
    T* Vt = Kt + (size_t)bk * row_k;

    for (int i = threadIdx.x; i < H * H; i += TALK_THREADS) mix[i] = p.talk[i] * p.temp[i % H] * p.scale;
    for (int i = threadIdx.x; i < BQ * H; i += TALK_THREADS) {
        const bool opens = p.sink && !split;            // (a split's rows open empty: the merge brings the sink in)
        run_m[i] = opens ? p.sink[i % H] : -INFINITY;   // the sink opens every row: maximum sink_h, sum exp(sink_h - sink_h) = 1
        run_l[i] = opens ? 1.f : 0.f;
    }
    const T* qsrc = (const T*)p.q + (size_t)(tok0 + q0) * hd;
    for (int i = threadIdx.x; i < BQ * hd; i += TALK_THREADS) {
        Q[i] = i < nq * hd ? to_float(qsrc[i]) : 0.f;
        O[i] = 0.f;
    }
    const int lo = lowest_seen(pos_first, p.mask_kind, p.mask_size);
    const int* table = p.block_table + (size_t)slot * p.table_stride;
    int k_begin = lo / bk * bk, k_end = pos_last;
    if (split) {
        k_begin += blockIdx.x * p.split_keys;
        k_end = min(k_end, k_begin + p.split_keys - 1);
    }
    for (int k0 = k_begin; k0 <= k_end; k0 += bk) {
        __syncthreads();   // the tiles and scores of the tile before are no longer read; first tile: Q, O, mix are written
        // -- the key and value tiles: row kj holds position k0 + kj for all key heads; rows that no query of the block sees are zeros
        {
            const int block = table[k0 / p.block_tokens];
            const int off = k0 % p.block_tokens;
            // eight threads a key row (a row's pieces are shared out among them, head by head)
            for (int kj = threadIdx.x >> 3; kj < bk; kj += TALK_THREADS >> 3) {
                const int pos = k0 + kj;
                const bool live_row = pos >= lo && pos <= pos_last && block >= 0;
                for (int g = 0; g < G; g++) {
                    const size_t src = (((size_t)(live_row ? block : 0) * G + g) * p.block_tokens + off + kj) * d;
                    for (int x = (threadIdx.x & 7) * VEC; x < d; x += 8 * VEC) {
                        Pack<T, VEC> kv, vv;
                        if (live_row) {
                            kv = load_pack<T, VEC>((const T*)p.k_cache + src + x);
                            vv = load_pack<T, VEC>((const T*)p.v_cache + src + x);
                        } else {
#pragma unroll
                            for (int z = 0; z < VEC; z++) kv.v[z] = vv.v[z] = from_float<T>(0.f);
                        }
                        store_pack<T, VEC>(Kt + (size_t)kj * row_k + (size_t)g * d + x, kv);
                        store_pack<T, VEC>(Vt + (size_t)kj * row_k + (size_t)g * d + x, vv);
                    }
                }
            }
        }
        __syncthreads();
        // -- raw scores: an item is (head, key); the key's entries are read once for all BQ queries
        for (int item = threadIdx.x; item < H * bk; item += TALK_THREADS) {
            const int h = item / bk, kj = item - h * bk;
            const T* kr = Kt + (size_t)kj * row_k + (size_t)(h / rep) * d;
            const float* qh = Q + (size_t)h * d;
            float acc[BQ];
#pragma unroll
            for (int qi = 0; qi < BQ; qi++) acc[qi] = 0.f;
            if constexpr (BQ == 1 && VEC > 1) {       // one query: VEC sums side by side instead of one long chain
                float part[VEC];
#pragma unroll
                for (int z = 0; z < VEC; z++) part[z] = 0.f;
#pragma unroll 4
                for (int e = 0; e < d; e += VEC) {
                    const Pack<T, VEC> kv = load_pack<T, VEC>(kr + e);
#pragma unroll
                    for (int z = 0; z < VEC; z += 4) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qh + e + z);      // (Q rows start on 16 bytes; VEC is 4 or 8)
                        part[z] = fmaf(q4.x, to_float(kv.v[z]), part[z]);
                        part[z + 1] = fmaf(q4.y, to_float(kv.v[z + 1]), part[z + 1]);
                        part[z + 2] = fmaf(q4.z, to_float(kv.v[z + 2]), part[z + 2]);
                        part[z + 3] = fmaf(q4.w, to_float(kv.v[z + 3]), part[z + 3]);
                    }
                }
#pragma unroll
                for (int z = 0; z < VEC; z++) acc[0] += part[z];
            } else {
                for (int e = 0; e < d; e += VEC) {
                    const Pack<T, VEC> kv = load_pack<T, VEC>(kr + e);
                    float kf[VEC];
#pragma unroll
                    for (int z = 0; z < VEC; z++) kf[z] = to_float(kv.v[z]);
#pragma unroll
                    for (int qi = 0; qi < BQ; qi++) {
                        const float* qq = qh + (size_t)qi * hd + e;
#pragma unroll
                        for (int z = 0; z < VEC; z++) acc[qi] = fmaf(qq[z], kf[z], acc[qi]);
                    }
                }
            }
#pragma unroll
            for (int qi = 0; qi < BQ; qi++) s_raw[((size_t)qi * H + h) * bk + kj] = acc[qi];
        }
        __syncthreads();
        // -- the heads talk; then the mask
        for (int item = threadIdx.x; item < BQ * H * bk; item += TALK_THREADS) {
            const int kj = item % bk, h = (item / bk) % H, qi = item / (bk * H);
            const float* rw = s_raw + (size_t)qi * H * bk + kj;
            const float* mh = mix + (size_t)h * H;
            float s = 0.f;
            for (int g = 0; g < H; g++) s = fmaf(mh[g], rw[(size_t)g * bk], s);
            const int qpos = pos_first + qi, kpos = k0 + kj;
            const bool seen = qi < nq && kpos <= qpos && kpos >= lowest_seen(qpos, p.mask_kind, p.mask_size);
            s_mix[item] = seen ? s : -INFINITY;
        }
        __syncthreads();
        // -- running softmax: a warp takes a row (query, head), a lane a key
        {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            for (int row = warp; row < BQ * H; row += TALK_THREADS / 32) {
                const float s = lane < bk ? s_mix[(size_t)row * bk + lane] : -INFINITY;
                const float m_old = run_m[row];
                const float m_new = fmaxf(m_old, warp_max(s));
                const float pr = (m_new == -INFINITY || s == -INFINITY) ? 0.f : expf(s - m_new);
                const float sum = warp_sum(pr);
                if (lane < bk) s_mix[(size_t)row * bk + lane] = pr;
                if (lane == 0) {
                    const float a = m_new == -INFINITY ? 1.f : (m_old == -INFINITY ? 0.f : expf(m_old - m_new));
                    alpha[row] = a;
                    run_l[row] = run_l[row] * a + sum;
                    run_m[row] = m_new;
                }
            }
        }
        __syncthreads();
        // -- O = alpha O + P V.  Few queries a block: an item is (head, VEC neighbouring value entries), read in one access a key;
        //    many: an item is (head, value entry), a value read once for all BQ queries
        if constexpr (VEC > 1 && BQ * VEC <= 32) {
            for (int item = threadIdx.x; item < hd / VEC; item += TALK_THREADS) {
                const int e0 = item * VEC, h = e0 / d, c = e0 - h * d;
                const T* vc = Vt + (size_t)(h / rep) * d + c;
                const float* ph = s_mix + (size_t)h * bk;
                float acc[BQ][VEC];
#pragma unroll
                for (int qi = 0; qi < BQ; qi++)
#pragma unroll
                    for (int z = 0; z < VEC; z++) acc[qi][z] = 0.f;
#pragma unroll 4
                for (int kj = 0; kj < bk; kj++) {
                    const Pack<T, VEC> vv = load_pack<T, VEC>(vc + (size_t)kj * row_k);
#pragma unroll
                    for (int qi = 0; qi < BQ; qi++) {
                        const float pw = ph[(size_t)qi * H * bk + kj];
#pragma unroll
                        for (int z = 0; z < VEC; z++) acc[qi][z] = fmaf(pw, to_float(vv.v[z]), acc[qi][z]);
                    }
                }
#pragma unroll
                for (int qi = 0; qi < BQ; qi++) {
                    float* o = O + (size_t)qi * hd + e0;
                    const float a = alpha[qi * H + h];
#pragma unroll
                    for (int z = 0; z < VEC; z++) o[z] = o[z] * a + acc[qi][z];
                }
            }
        } else {
            for (int item = threadIdx.x; item < hd; item += TALK_THREADS) {
                const int h = item / d, c = item - h * d;
                const T* vc = Vt + (size_t)(h / rep) * d + c;
                const float* ph = s_mix + (size_t)h * bk;
                float acc[BQ];
#pragma unroll
                for (int qi = 0; qi < BQ; qi++) acc[qi] = 0.f;
#pragma unroll 8
                for (int kj = 0; kj < bk; kj++) {
                    const float v = to_float(vc[(size_t)kj * row_k]);
#pragma unroll
                    for (int qi = 0; qi < BQ; qi++) acc[qi] = fmaf(ph[(size_t)qi * H * bk + kj], v, acc[qi]);
                }
#pragma unroll
                for (int qi = 0; qi < BQ; qi++) {
                    float* o = O + (size_t)qi * hd + item;
                    *o = *o * alpha[qi * H + h] + acc[qi];
                }
            }
        }
    }
    __syncthreads();
    if (split) {
        for (int i = threadIdx.x; i < hd; i += TALK_THREADS) my_o[i] = O[i];
        for (int i = threadIdx.x; i < H; i += TALK_THREADS) { my_ml[i] = run_m[i]; my_ml[H + i] = run_l[i]; }
        return;
    }
    const T* gate = p.gate ? (const T*)p.gate + (size_t)(tok0 + q0) * p.ldg : nullptr;
    for (int i = threadIdx.x; i < nq * hd; i += TALK_THREADS) {
        const int qi = i / hd, e = i - qi * hd;
        const float l = run_l[qi * H + e / d];
        float v = l > 0.f ? O[i] / l : 0.f;
        if (gate) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)qi * p.ldg + e])));
        out[i] = from_float<T>(v);
    }
}

// What the splits of a decode step left, folded: with M_h = max(sink_h, the splits' maxima),
//   out[e] = sum_s exp(m_s - M) O_s[e] / (exp(sink_h - M) + sum_s exp(m_s - M) l_s)  [* sigmoid(gate[e])],   h = the head of entry e.
// A block a sequence; the splits are added in their order.
template <typename T>
__global__ void __launch_bounds__(256)
talk_merge_kernel(T* __restrict__ out, const T* __restrict__ gate, long ldg, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                  const float* __restrict__ sink, const int* __restrict__ slot_ids, const int* __restrict__ cu_seqlens, int heads, int d,
                  int max_splits) {
    extern __shared__ float wsm[];      // [max_splits][heads] weights, then [heads] 1 / denominators
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x, hd = heads * d;
    const int tok = cu_seqlens[b];
    if (cu_seqlens[b + 1] - tok <= 0) return;      // (a sequence without a token in this step)
    T* o = out + (size_t)tok * hd;
    if (slot_ids[b] < 0) {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) o[i] = from_float<T>(0.f);
        return;
    }
    const float* ml = part_ml + (size_t)b * max_splits * 2 * heads;
    float* inv = wsm + max_splits * heads;
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        float M = sink ? sink[h] : -INFINITY;
        for (int s = 0; s < max_splits; s++) M = fmaxf(M, ml[(size_t)s * 2 * heads + h]);
        float den = (sink && M != -INFINITY) ? expf(sink[h] - M) : 0.f;
        for (int s = 0; s < max_splits; s++) {
            const float m = ml[(size_t)s * 2 * heads + h];
            const float w = (m == -INFINITY || M == -INFINITY) ? 0.f : expf(m - M);
            wsm[s * heads + h] = w;
            den = fmaf(w, ml[(size_t)s * 2 * heads + heads + h], den);
        }
        inv[h] = den > 0.f ? 1.0f / den : 0.f;
    }
    __syncthreads();
    const float* po = part_o + (size_t)b * max_splits * hd;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        const int h = e / d;
        float v = 0.f;
        for (int s = 0; s < max_splits; s++) {
            const float w = wsm[s * heads + h];
            if (w != 0.f) v = fmaf(w, po[(size_t)s * hd + e], v);     // (a split without keys left nothing to read)
        }
        v *= inv[h];
        if (gate) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)tok * ldg + e])));
        o[e] = from_float<T>(v);
    }
}

size_t talk_smem_bytes(int bq, int bk, int heads, int kv_heads, int d, int vec, size_t es) {
    const size_t floats = (size_t)heads * heads + heads + 3 * (size_t)bq * heads + 4 + 2 * (size_t)bq * heads * d + 2 * (size_t)bq * heads * bk;
    return floats * 4 + 2 * (size_t)bk * ((size_t)kv_heads * d + vec) * es;
}

template <typename T, int BQ, int VEC>
cudaError_t talk_launch(const TalkParams& p, int max_new_tokens, int batch, size_t smem, cudaStream_t stream) {
    auto kernel = talking_attention_kernel<T, BQ, VEC>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int tiles = p.split_keys > 0 ? p.max_splits : (max_new_tokens + BQ - 1) / BQ;
    cudaError_t e = launch_pdl(kernel, dim3(tiles, batch), dim3(TALK_THREADS), smem, stream, p);
    if (e != cudaSuccess || p.split_keys == 0) return e;
    const size_t msm = sizeof(float) * ((size_t)p.max_splits * p.heads + p.heads);
    return launch_pdl(talk_merge_kernel<T>, dim3(batch), dim3(256), msm, stream, (T*)p.out, (const T*)p.gate, p.ldg, (const float*)p.part_o,
                      (const float*)p.part_ml, p.sink, p.slot_ids, p.cu_seqlens, p.heads, p.d, p.max_splits);
}

}  // namespace

HYMT2_API int hymt2_talk_prep(const void* x, long ldx, int dtype, void* q_out, void* k_cache, void* v_cache, const int* block_table,
                              int table_stride, int block_tokens, const int* token_seq, const int* token_pos, const int* slot_ids,
                              const float* inv_freq, int rot_dims, int tokens, int heads, int kv_heads, int d, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0 && d > 0 && block_tokens > 0, "talk_prep: bad sizes");
    HYMT2_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= d, "talk_prep: %d rotated entries of %d", rot_dims, d);
    HYMT2_REQUIRE(rot_dims == 0 || inv_freq != nullptr, "talk_prep: no frequencies");
    TalkPrepParams p;
    p.x = x; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.token_seq = token_seq;
    p.token_pos = token_pos; p.slot_ids = slot_ids; p.inv_freq = inv_freq; p.ldx = ldx; p.table_stride = table_stride;
    p.block_tokens = block_tokens; p.heads = heads; p.kv_heads = kv_heads; p.d = d; p.rot_dims = rot_dims;
    HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(talk_prep_kernel<T>, dim3(tokens), dim3(128), sizeof(float) * (size_t)(rot_dims + 2), stream, p));
    return hymt2_check_launch("talk_prep");
}

HYMT2_API int hymt2_talking_attention(void* out, const void* q, const void* gate, long ldg, const void* k_cache, const void* v_cache, int dtype,
                                      const int* block_table, int table_stride, int block_tokens, const int* cu_seqlens,
                                      const int* slot_ids, const int* kv_lens, int batch, int max_new_tokens, int heads, int kv_heads,
                                      int d, float scale, const float* talk, const float* temp, const float* sink, int mask_kind,
                                      int mask_size, int split_keys, int max_splits, float* part_o, float* part_ml, cudaStream_t stream) {
    if (batch == 0 || max_new_tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && max_new_tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && d > 0,
                  "talking_attention: bad sizes");
    HYMT2_REQUIRE(split_keys == 0 || (max_new_tokens == 1 && max_splits > 0 && max_splits <= 65535 && part_o && part_ml && split_keys % 32 == 0),
                  "talking_attention: splits are for steps of one token a sequence, in whole key tiles, with room for their sums");
    HYMT2_REQUIRE(mask_kind == MASK_NONE || (mask_size > 0 && (mask_kind == MASK_CHUNK || mask_kind == MASK_WINDOW)),
                  "talking_attention: mask kind %d with size %d", mask_kind, mask_size);
    HYMT2_REQUIRE(block_tokens > 0, "talking_attention: block_tokens must be positive");
    const size_t es = dtype == HYMT2_BF16 ? 2 : 4;
    const int full = (int)(16 / es);
    const bool aligned = d % full == 0 && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0;
    const int vec = aligned ? full : 1;
    // keys per tile: at most 32 (a lane a key in the softmax), a divisor of the cache's block
    int bk = 32;
    while (bk > 1 && block_tokens % bk) bk >>= 1;
    int dev = 0, limit = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    // queries per block: a decode step has one a sequence; a prompt takes 16, or 4 where 16 do not fit the shared memory
    int bq = max_new_tokens == 1 ? 1 : 16;
    while (true) {
        if (talk_smem_bytes(bq, bk, heads, kv_heads, d, vec, es) <= (size_t)limit) break;
        if (bq > 1) bq = bq == 16 ? 4 : 1;
        else if (bk > 4 && block_tokens % (bk / 2) == 0) bk >>= 1;
        else break;
    }
    const size_t smem = talk_smem_bytes(bq, bk, heads, kv_heads, d, vec, es);
    HYMT2_REQUIRE(smem <= (size_t)limit, "talking_attention: %d heads of %d entries do not fit the shared memory (%zu bytes)", heads, d, smem);
    TalkParams p;
    p.out = out; p.q = q; p.gate = gate; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.cu_seqlens = cu_seqlens;
    p.slot_ids = slot_ids; p.kv_lens = kv_lens; p.talk = talk; p.temp = temp; p.sink = sink; p.ldg = ldg; p.table_stride = table_stride;
    p.block_tokens = block_tokens; p.heads = heads; p.kv_heads = kv_heads; p.d = d; p.mask_kind = mask_kind; p.mask_size = mask_size;
    p.bk = bk; p.scale = scale;
    p.split_keys = split_keys; p.max_splits = max_splits; p.part_o = part_o; p.part_ml = part_ml;
    HYMT2_REQUIRE(split_keys == 0 || (bq == 1 && split_keys % bk == 0), "talking_attention: splits of %d keys do not fit tiles of %d", split_keys, bk);
    cudaError_t e = cudaSuccess;
#define TALK_GO(T, V)                                                                           \
    do {                                                                                        \
        if (bq == 16) e = talk_launch<T, 16, V>(p, max_new_tokens, batch, smem, stream);       \
        else if (bq == 4) e = talk_launch<T, 4, V>(p, max_new_tokens, batch, smem, stream);    \
        else e = talk_launch<T, 1, V>(p, max_new_tokens, batch, smem, stream);                 \
    } while (0)
    if (dtype == HYMT2_BF16) { if (vec == 8) TALK_GO(__nv_bfloat16, 8); else TALK_GO(__nv_bfloat16, 1); }
    else if (dtype == HYMT2_F32) { if (vec == 4) TALK_GO(float, 4); else TALK_GO(float, 1); }
    else { hymt2_set_error("unknown dtype code %d", dtype); return HYMT2_ERR_ARGUMENT; }
#undef TALK_GO
    if (e != cudaSuccess) { hymt2_set_error("talking_attention: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
    return hymt2_check_launch("talking_attention");
}
