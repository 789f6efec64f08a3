// The attention whose heads talk (see talking_attention.cu for the mechanism) for prompts in bfloat16, with its two
// products on the tensor cores through warp-level matrix fragments (16x16x16, float32 accumulation).
//
// A block owns 16 queries of one sequence and ALL heads, because the scores of every head at a (query, key) pair are mixed
// before the softmax.  It walks the keys that its queries see in tiles of 32 (a divisor of the cache's block, so that a tile is
// one contiguous piece of a block).  Per tile:
//   raw_g = Q_g K_g^T       fragments into shared memory, float32                                  (tensor cores)
//   s_h = sum_g talk[h, g] * temp[g] * scale * raw_g; the mask          a thread per (query, key) pair, float32, in place
//   running softmax per (head, query) row; the weights rounded to bfloat16 as the second product's operand
//   O_h = O_h * shrink + P_h V_g                          O in accumulator fragments, a warp holds whole heads' pieces
// The sink opens every row (running maximum sink_h, running sum 1).  How the entries of an accumulator fragment map to rows is
// found out once, by loading a matrix whose entries are their own row numbers.  Values are another plane than keys.
#include "common.cuh"

#include <mma.h>

namespace {

using namespace nvcuda;
typedef __nv_bfloat16 bf16;

constexpr int TM_BQ = 16, TM_BK = 32, TM_MAXH = 16, TM_SLD = TM_BK + 4, TM_PLD = TM_BK + 8, TM_XLD = 20;
enum { TM_MASK_NONE = 0, TM_MASK_CHUNK = 1, TM_MASK_WINDOW = 2 };

struct TalkMmaParams {
    bf16* out;             // [T, heads * d]
    const bf16* q;         // [T, heads * d]
    const bf16* gate;      // [T, ldg] or null
    const bf16* k_cache;
    const bf16* v_cache;
    const int* block_table;
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    const float* talk;
    const float* temp;
    const float* sink;
    long ldg;
    int table_stride, block_tokens, heads, kv_heads, d, mask_kind, mask_size;
    float scale;
};

// 16 bytes from global to shared memory without a stop in registers; `valid` false: 16 zero bytes (nothing is read, the address
// only has to be one that exists).  Copies are committed in groups; tm_wait_but_one leaves the newest group in flight.
__device__ __forceinline__ void tm_copy16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tm_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

__device__ __forceinline__ int tm_lowest_seen(int pos, int kind, int size) {
    if (kind == TM_MASK_CHUNK) return pos / size * size;
    if (kind == TM_MASK_WINDOW) return max(0, pos - size + 1);
    return 0;
}

size_t tm_smem_bytes(int H, int G, int d, int warps) {
    const size_t ldq = (size_t)H * d + 8, ldk = (size_t)G * d + 8;
    return 2 * (TM_BQ * ldq + 2 * TM_BK * ldk + (size_t)H * TM_BQ * TM_PLD) + 4 * ((size_t)H * TM_BQ * TM_SLD + (size_t)warps * 16 * TM_XLD + (size_t)H * TM_MAXH + 3 * (size_t)H * TM_BQ) + 128;
}

// MAXF: the most output fragments (a head's 16 queries x 16 value entries) that a warp holds
template <int MAXF, int TM_THREADS>
__global__ void __launch_bounds__(TM_THREADS)
talking_attention_mma_kernel(TalkMmaParams p) {
    constexpr int TM_WARPS = TM_THREADS / 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.y;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    // (the tiles with the most keys first: a chunk's last queries see all of it)
    const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * TM_BQ;
    if (q0 >= n) return;
    const int nq = min(TM_BQ, n - q0);
    const int slot = p.slot_ids[b];
    const int H = p.heads, G = p.kv_heads, d = p.d, rep = H / G, hd = H * d, gd = G * d;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bf16* out = p.out + (size_t)(tok0 + q0) * hd;
    if (slot < 0) {
        for (int i = tid; i < nq * hd; i += TM_THREADS) out[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int ldq = hd + 8, ldk = gd + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][ldq]
    bf16* Ks = Qs + TM_BQ * ldq;                                  // [32][ldk]
    bf16* Vs = Ks + TM_BK * ldk;                                  // [32][ldk]
    bf16* Ps = Vs + TM_BK * ldk;                                  // [H][16][TM_PLD]
    float* Ss = reinterpret_cast<float*>(Ps + (size_t)H * TM_BQ * TM_PLD);   // [H][16][TM_SLD]
    float* Xs = Ss + (size_t)H * TM_BQ * TM_SLD;                  // [8 warps][16][TM_XLD]: a fragment on its way out
    float* mix = Xs + TM_WARPS * 16 * TM_XLD;                     // [H][16]: talk[h, g] * temp[g] * scale, zeros behind the last head
    float* run_m = mix + H * TM_MAXH;                                   // [H][16]
    float* run_l = run_m + H * TM_BQ;
    float* shrink = run_l + H * TM_BQ;

    const int start = p.kv_lens[b] - n;
    const int pos_first = start + q0, pos_last = start + q0 + nq - 1;
    for (int i = tid; i < H * TM_MAXH; i += TM_THREADS) {
        const int h = i / TM_MAXH, g = i % TM_MAXH;
        mix[i] = g < H ? p.talk[h * H + g] * p.temp[g] * p.scale : 0.f;
    }
    for (int i = tid; i < H * TM_BQ; i += TM_THREADS) {
        run_m[i] = p.sink ? p.sink[i / TM_BQ] : -INFINITY;
        run_l[i] = p.sink ? 1.f : 0.f;
    }
    {   // the queries, 16 bytes a piece; rows behind the last live one are zeros
        const bf16* qg = p.q + (size_t)(tok0 + q0) * hd;
        const int per_row = hd / 8;
        for (int i = tid; i < TM_BQ * per_row; i += TM_THREADS) {
            const int r = i / per_row, c = (i - r * per_row) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < nq) v = *reinterpret_cast<const uint4*>(qg + (size_t)r * hd + c);
            *reinterpret_cast<uint4*>(Qs + r * ldq + c) = v;
        }
    }
    const int lo = tm_lowest_seen(pos_first, p.mask_kind, p.mask_size);
    const int* table = p.block_table + (size_t)slot * p.table_stride;
    // which of its 16 rows each entry of an accumulator fragment belongs to
    float* xw = Xs + warp * 16 * TM_XLD;
    for (int i = lane; i < 256; i += 32) xw[(i >> 4) * TM_XLD + (i & 15)] = (float)(i >> 4);
    __syncwarp();
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[MAXF];
    int row_of[8];
    {
        wmma::load_matrix_sync(acc[0], xw, TM_XLD, wmma::mem_row_major);
#pragma unroll
        for (int e = 0; e < 8; e++) row_of[e] = (int)acc[0].x[e];
    }
    // (the entries of a thread lie in two rows in the layouts known; found out, not assumed)
    int other_row = row_of[0];
    bool two_rows = true;
#pragma unroll
    for (int e = 1; e < 8; e++)
        if (row_of[e] != row_of[0]) {
            if (other_row == row_of[0]) other_row = row_of[e];
            else if (row_of[e] != other_row) two_rows = false;
        }
#pragma unroll
    for (int i = 0; i < MAXF; i++) wmma::fill_fragment(acc[i], 0.f);
    const int dblocks = d / 16, frags = H * dblocks;
    const int per_warp = (frags + TM_WARPS - 1) / TM_WARPS;       // <= MAXF; a warp's fragments are neighbours: few heads a warp
    const int f0 = warp * per_warp;

    // A tile of keys or of values on its way into shared memory: eight threads a row, 16 bytes a piece; a row that no query of
    // the block sees is zeros.  The key tile of pass n + 1 is asked for as soon as pass n's scores are made, the value tile
    // of pass n at its start: both arrive under the other work of the pass.
    auto ask_tile = [&](bf16* dst, const bf16* cache, int k0) {
        if (k0 <= pos_last) {
            const int block = table[k0 / p.block_tokens], off = k0 % p.block_tokens;
            constexpr int PER_ROW = TM_THREADS / TM_BK;          // threads that share a key row
            const int kj = tid / PER_ROW, pos = k0 + kj;
            const bool live_row = pos >= lo && pos <= pos_last && block >= 0;
            for (int g = 0; g < G; g++) {
                const bf16* src = cache + (((size_t)(live_row ? block : 0) * G + g) * p.block_tokens + off + kj) * d;
                bf16* row = dst + kj * ldk + g * d;
                for (int x = (tid % PER_ROW) * 8; x < d; x += PER_ROW * 8) tm_copy16(row + x, src + x, live_row);
            }
        }
        tm_commit();
    };
    const int k_first = lo / TM_BK * TM_BK;
    ask_tile(Ks, p.k_cache, k_first);
    for (int k0 = k_first; k0 <= pos_last; k0 += TM_BK) {
        __syncthreads();   // the value tile and the weights of the pass before are no longer read (first pass: Q, mix, the rows' openings)
        ask_tile(Vs, p.v_cache, k0);
        tm_wait_but_one();  // the keys of this pass are here (the values may still be on their way)
        __syncthreads();
        // -- raw scores: with eight warps a warp takes a head and both halves of the key tile share the head's query fragments;
        //    with sixteen a warp takes one half of a head's tile
        if constexpr (TM_WARPS <= 8) {
            for (int h = warp; h < H; h += TM_WARPS) {
                wmma::fragment<wmma::accumulator, 16, 16, 16, float> s0, s1;
                wmma::fill_fragment(s0, 0.f);
                wmma::fill_fragment(s1, 0.f);
                const bf16* qh = Qs + h * d;
                const bf16* kh = Ks + (h / rep) * d;
                for (int ks = 0; ks < dblocks; ks++) {
                    wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b0, b1;
                    wmma::load_matrix_sync(a, qh + ks * 16, ldq);
                    wmma::load_matrix_sync(b0, kh + ks * 16, ldk);
                    wmma::load_matrix_sync(b1, kh + 16 * ldk + ks * 16, ldk);
                    wmma::mma_sync(s0, a, b0, s0);
                    wmma::mma_sync(s1, a, b1, s1);
                }
                wmma::store_matrix_sync(Ss + (size_t)h * TM_BQ * TM_SLD, s0, TM_SLD, wmma::mem_row_major);
                wmma::store_matrix_sync(Ss + (size_t)h * TM_BQ * TM_SLD + 16, s1, TM_SLD, wmma::mem_row_major);
            }
        } else {
            for (int item = warp; item < 2 * H; item += TM_WARPS) {
                const int h = item >> 1, kb = item & 1;
                wmma::fragment<wmma::accumulator, 16, 16, 16, float> s0;
                wmma::fill_fragment(s0, 0.f);
                const bf16* qh = Qs + h * d;
                const bf16* kh = Ks + (h / rep) * d + kb * 16 * ldk;
                for (int ks = 0; ks < dblocks; ks++) {
                    wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b0;
                    wmma::load_matrix_sync(a, qh + ks * 16, ldq);
                    wmma::load_matrix_sync(b0, kh + ks * 16, ldk);
                    wmma::mma_sync(s0, a, b0, s0);
                }
                wmma::store_matrix_sync(Ss + (size_t)h * TM_BQ * TM_SLD + kb * 16, s0, TM_SLD, wmma::mem_row_major);
            }
        }
        __syncthreads();
        ask_tile(Ks, p.k_cache, k0 + TM_BK);   // the key tile is free: the keys of the next pass (or an empty group behind the last pass)
        // -- the heads talk; then the mask.  A thread owns a (query, key) pair across all heads, so the mixing is in place.
        for (int pair = tid; pair < TM_BQ * TM_BK; pair += TM_THREADS) {
            const int qi = pair / TM_BK, kj = pair % TM_BK;
            float raw[TM_MAXH];
#pragma unroll
            for (int g = 0; g < TM_MAXH; g++) raw[g] = g < H ? Ss[((size_t)g * TM_BQ + qi) * TM_SLD + kj] : 0.f;
            const int qpos = pos_first + qi, kpos = k0 + kj;
            const bool seen = qi < nq && kpos <= qpos && kpos >= tm_lowest_seen(qpos, p.mask_kind, p.mask_size);
            for (int h = 0; h < H; h++) {
                const float4* mh = reinterpret_cast<const float4*>(mix + h * TM_MAXH);      // (rows of 16, zeros behind the last head)
                float s = 0.f;
#pragma unroll
                for (int g4 = 0; g4 < TM_MAXH / 4; g4++)
                    if (g4 * 4 < H) {
                        const float4 m4 = mh[g4];
                        s = fmaf(m4.x, raw[4 * g4], fmaf(m4.y, raw[4 * g4 + 1], fmaf(m4.z, raw[4 * g4 + 2], fmaf(m4.w, raw[4 * g4 + 3], s))));
                    }
                Ss[((size_t)h * TM_BQ + qi) * TM_SLD + kj] = seen ? s : -INFINITY;
            }
        }
        __syncthreads();
        // -- running softmax: a thread takes a row (head, query) and walks its 32 keys
        for (int row = tid; row < H * TM_BQ; row += TM_THREADS) {
            float* sr = Ss + (size_t)row * TM_SLD;
            const float m_old = run_m[row];
            float m_new = m_old;
#pragma unroll
            for (int j = 0; j < TM_BK; j += 4) {
                const float4 v = *reinterpret_cast<const float4*>(sr + j);
                m_new = fmaxf(fmaxf(m_new, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
            }
            float sum = 0.f;
            bf16* pr = Ps + (size_t)row * TM_PLD;
#pragma unroll
            for (int j = 0; j < TM_BK; j += 4) {
                const float4 v = *reinterpret_cast<const float4*>(sr + j);
                float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int z = 0; z < 4; z++) {
                    e[z] = (m_new == -INFINITY || e[z] == -INFINITY) ? 0.f : expf(e[z] - m_new);
                    sum += e[z];
                }
                __nv_bfloat162 h2[2] = {__floats2bfloat162_rn(e[0], e[1]), __floats2bfloat162_rn(e[2], e[3])};
                *reinterpret_cast<uint2*>(pr + j) = *reinterpret_cast<const uint2*>(h2);
            }
            const float a = m_new == -INFINITY ? 1.f : (m_old == -INFINITY ? 0.f : expf(m_old - m_new));
            shrink[row] = a;
            run_l[row] = run_l[row] * a + sum;
            run_m[row] = m_new;
        }
        tm_wait_but_one();   // the values of this pass are here (the keys of the next pass may still be on their way)
        __syncthreads();
        // -- O = shrink O + P V
        {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> pa0, pa1;
            int loaded = -1;
#pragma unroll
            for (int i = 0; i < MAXF; i++) {
                const int f = f0 + i;
                if (i < per_warp && f < frags) {
                    const int h = f / dblocks, db = f - h * dblocks;
                    if (h != loaded) {
                        wmma::load_matrix_sync(pa0, Ps + (size_t)h * TM_BQ * TM_PLD, TM_PLD);
                        wmma::load_matrix_sync(pa1, Ps + (size_t)h * TM_BQ * TM_PLD + 16, TM_PLD);
                        loaded = h;
                    }
                    if (two_rows) {
                        const float sa = shrink[h * TM_BQ + row_of[0]], sb = shrink[h * TM_BQ + other_row];
#pragma unroll
                        for (int e = 0; e < 8; e++) acc[i].x[e] *= row_of[e] == row_of[0] ? sa : sb;
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; e++) acc[i].x[e] *= shrink[h * TM_BQ + row_of[e]];
                    }
                    const bf16* vh = Vs + (h / rep) * d + db * 16;
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> v0, v1;
                    wmma::load_matrix_sync(v0, vh, ldk);
                    wmma::load_matrix_sync(v1, vh + 16 * ldk, ldk);
                    wmma::mma_sync(acc[i], pa0, v0, acc[i]);
                    wmma::mma_sync(acc[i], pa1, v1, acc[i]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    const bf16* gate = p.gate ? p.gate + (size_t)(tok0 + q0) * p.ldg : nullptr;
#pragma unroll
    for (int i = 0; i < MAXF; i++) {
        const int f = f0 + i;
        if (i < per_warp && f < frags) {
            const int h = f / dblocks, db = f - h * dblocks;
            wmma::store_matrix_sync(xw, acc[i], TM_XLD, wmma::mem_row_major);
            __syncwarp();
            for (int e = lane; e < 256; e += 32) {
                const int r = e >> 4, c = e & 15;
                if (r < nq) {
                    const float l = run_l[h * TM_BQ + r];
                    float v = l > 0.f ? xw[r * TM_XLD + c] / l : 0.f;
                    const int col = h * d + db * 16 + c;
                    if (gate) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * p.ldg + col])));
                    out[(size_t)r * hd + col] = __float2bfloat16_rn(v);
                }
            }
            __syncwarp();
        }
    }
}

template <int MAXF, int THREADS>
cudaError_t tm_launch(const TalkMmaParams& p, int max_new_tokens, int batch, size_t smem, cudaStream_t stream) {
    auto kernel = talking_attention_mma_kernel<MAXF, THREADS>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(kernel, dim3((max_new_tokens + TM_BQ - 1) / TM_BQ, batch), dim3(THREADS), smem, stream, p);
}

}  // namespace

// 1 if the tensor-core form takes these sizes (bfloat16 only): heads of a multiple of 16 entries, at most 16 heads, cache
// blocks in whole key tiles, and everything of a block within the shared memory
HYMT2_API int hymt2_talking_attention_mma_supported(int heads, int kv_heads, int d, int block_tokens) {
    if (heads < 1 || heads > TM_MAXH || kv_heads < 1 || heads % kv_heads || d < 16 || d % 16 || block_tokens % TM_BK) return 0;
    if ((heads * (d / 16) + 7) / 8 > 16) return 0;
    int dev = 0, limit = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    return tm_smem_bytes(heads, kv_heads, d, 8) <= (size_t)limit ? 1 : 0;
}

HYMT2_API int hymt2_talking_attention_mma(void* out, const void* q, const void* gate, long ldg, const void* k_cache, const void* v_cache,
                                          const int* block_table, int table_stride, int block_tokens, const int* cu_seqlens,
                                          const int* slot_ids, const int* kv_lens, int batch, int max_new_tokens, int heads, int kv_heads,
                                          int d, float scale, const float* talk, const float* temp, const float* sink, int mask_kind,
                                          int mask_size, cudaStream_t stream) {
    if (batch == 0 || max_new_tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && max_new_tokens > 0, "talking_attention_mma: bad sizes");
    HYMT2_REQUIRE(hymt2_talking_attention_mma_supported(heads, kv_heads, d, block_tokens), "talking_attention_mma: %d heads on %d of %d entries, blocks of %d tokens: not taken", heads, kv_heads, d, block_tokens);
    HYMT2_REQUIRE(mask_kind == TM_MASK_NONE || (mask_size > 0 && (mask_kind == TM_MASK_CHUNK || mask_kind == TM_MASK_WINDOW)),
                  "talking_attention_mma: mask kind %d with size %d", mask_kind, mask_size);
    HYMT2_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0, "talking_attention_mma: operands must be 16-byte aligned");
    TalkMmaParams p;
    p.out = (bf16*)out; p.q = (const bf16*)q; p.gate = (const bf16*)gate; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.block_table = block_table; p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens; p.talk = talk; p.temp = temp;
    p.sink = sink; p.ldg = ldg; p.table_stride = table_stride; p.block_tokens = block_tokens; p.heads = heads; p.kv_heads = kv_heads; p.d = d;
    p.mask_kind = mask_kind; p.mask_size = mask_size; p.scale = scale;
    // sixteen warps a block where there is work for them (32 output fragments or more, at most 8 a warp) and room in the shared
    // memory; else eight
    const int frags = heads * (d / 16);
    int dev = 0, limit = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const bool wide = frags >= 32 && (frags + 15) / 16 <= 8 && tm_smem_bytes(heads, kv_heads, d, 16) <= (size_t)limit;
    const int warps = wide ? 16 : 8;
    const size_t smem = tm_smem_bytes(heads, kv_heads, d, warps);
    const int per_warp = (frags + warps - 1) / warps;
    cudaError_t e;
    if (wide) {
        if (per_warp <= 2) e = tm_launch<2, 512>(p, max_new_tokens, batch, smem, stream);
        else if (per_warp <= 4) e = tm_launch<4, 512>(p, max_new_tokens, batch, smem, stream);
        else e = tm_launch<8, 512>(p, max_new_tokens, batch, smem, stream);
    } else if (per_warp <= 2) e = tm_launch<2, 256>(p, max_new_tokens, batch, smem, stream);
    else if (per_warp <= 4) e = tm_launch<4, 256>(p, max_new_tokens, batch, smem, stream);
    else if (per_warp <= 8) e = tm_launch<8, 256>(p, max_new_tokens, batch, smem, stream);
    else e = tm_launch<16, 256>(p, max_new_tokens, batch, smem, stream);
    if (e != cudaSuccess) { hymt2_set_error("talking_attention_mma: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
    return hymt2_check_launch("talking_attention_mma");
}
