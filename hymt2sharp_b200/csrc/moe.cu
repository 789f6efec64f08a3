// Routing of a mixture of experts: from the router's outputs to the chosen experts and their weights, from there to
// the rows sorted by expert that the grouped products read, and from the experts' outputs back to one row per token.
// Everything here is float32 and integer arithmetic; nothing depends on the order in which blocks run (no atomics), so a
// token's result does not depend on what else is in the step.
//
//   route    scores s = softmax(z + bias) over ALL router outputs (bias: optional); the `top` largest of s + correction are
//            chosen (ties: the lower index); a chosen output's weight is its s, without the correction, either as it is or
//            (`renorm`) divided by the sum over the chosen ones, which is the softmax over the chosen outputs alone
//   count    how many (token, choice) pairs name each expert that has tensors (outputs from `experts` on name identity
//            experts, which need no product)
//   place    every expert's pairs, in token order, get consecutive rows of a sorted list; an expert's segment is padded to
//            whole tiles of `tile` rows.  Written: pair_row[pair] (-1 for identity experts), row_token[row] (-1 for padding),
//            tile_group[tile] (-1 for tiles not in use; the tiles in use come first, and their number follows the last entry)
//   combine  out[t] = sum over the token's choices, in the order they were chosen, of weight * (the expert's output row, or
//            the token's own input row for an identity expert)
#include "common.cuh"

namespace {

constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(int* __restrict__ chosen, float* __restrict__ weight, const float* __restrict__ logits,
                 const float* __restrict__ correction, const float* __restrict__ bias, int renorm, int tokens, int outputs, int top) {
    extern __shared__ float smem[];   // [ROUTE_WARPS][2 * outputs]: scores, choice scores
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= tokens) return;
    float* s = smem + (size_t)warp * 2 * outputs;
    float* c = s + outputs;
    const float* z = logits + (size_t)t * outputs;
    float m = -INFINITY;
    for (int i = lane; i < outputs; i += 32) m = fmaxf(m, z[i] + (bias ? bias[i] : 0.f));
    m = warp_max(m);
    float sum = 0.f;
    for (int i = lane; i < outputs; i += 32) { const float e = expf(z[i] + (bias ? bias[i] : 0.f) - m); s[i] = e; sum += e; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int i = lane; i < outputs; i += 32) {
        s[i] *= inv;
        c[i] = s[i] + (correction ? correction[i] : 0.f);
    }
    __syncwarp();
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int i = lane; i < outputs; i += 32)
            if (c[i] > best) { best = c[i]; at = i; }   // ascending i: the first of equals stays
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0) {
            chosen[(size_t)t * top + k] = at;
            weight[(size_t)t * top + k] = s[at];
            c[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm && lane == 0) {   // the weights become the softmax over the chosen outputs alone: the same exponentials, another sum
        float chosen_sum = 0.f;
        for (int k = 0; k < top; k++) chosen_sum += weight[(size_t)t * top + k];
        for (int k = 0; k < top; k++) weight[(size_t)t * top + k] /= chosen_sum;
    }
}

constexpr int PLACE_THREADS = 256;

__global__ void __launch_bounds__(PLACE_THREADS)
moe_count_kernel(int* __restrict__ counts, const int* __restrict__ chosen, int pairs, int experts) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int e = blockIdx.x;
    int n = 0;
    if (e < experts) {   // (a mixture of identity experts only still runs one block, which finds nothing)
        // 16 bytes a load and four loads in flight: few blocks walk all pairs, and only their loads' latency costs
        const int quads = ((uintptr_t)chosen % 16 == 0) ? pairs / 4 : 0;
        const int4* c4 = reinterpret_cast<const int4*>(chosen);
#pragma unroll 4
        for (int i = threadIdx.x; i < quads; i += blockDim.x) {
            const int4 v = __ldg(c4 + i);
            n += (v.x == e) + (v.y == e) + (v.z == e) + (v.w == e);
        }
        for (int i = quads * 4 + threadIdx.x; i < pairs; i += blockDim.x) n += chosen[i] == e;
    }
    // (counts of up to 2^24 are exact in float32)
    const float total = block_sum((float)n, scratch);
    if (threadIdx.x == 0) counts[e] = (int)total;
}

constexpr int PLACE_CHUNK = 8192;   // pairs that go through shared memory at a time

__global__ void __launch_bounds__(PLACE_THREADS)
moe_place_kernel(int* __restrict__ pair_row, int* __restrict__ row_token, int* __restrict__ tile_group,
                 const int* __restrict__ counts, const int* __restrict__ chosen, int pairs, int top, int experts, int tile,
                 int max_tiles) {
    __shared__ int chunk[PLACE_CHUNK + PLACE_CHUNK / 32];   // one word of padding every 32: a thread's run starts in a bank of its own
    __shared__ int warp_total[PLACE_THREADS / 32];
    __shared__ int base_s;
    pdl_wait();
    pdl_launch_dependents();
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        int rows = 0;
        for (int i = 0; i < e; i++) rows += (counts[i] + tile - 1) / tile * tile;
        base_s = rows;
    }
    __syncthreads();
    const int base = base_s;
    int placed = 0;   // hits of the chunks so far
    for (int c0 = 0; c0 < pairs; c0 += PLACE_CHUNK) {
        const int n = min(PLACE_CHUNK, pairs - c0);
        __syncthreads();
#pragma unroll 8
        for (int i = threadIdx.x; i < n; i += blockDim.x) chunk[i + (i >> 5)] = __ldg(chosen + c0 + i);   // neighbours read neighbours
        __syncthreads();
        // A thread owns a run of consecutive pairs: it counts its hits, a scan over the threads' counts gives the place of
        // its first hit, and a second walk over the run writes the rows.  Pairs keep their order.
        const int run = (n + PLACE_THREADS - 1) / PLACE_THREADS;
        const int i0 = min(n, (int)threadIdx.x * run), i1 = min(n, i0 + run);
        int hits = 0;
        if (e < experts)
            for (int i = i0; i < i1; i++) hits += chunk[i + (i >> 5)] == e;
        int incl = hits;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) warp_total[warp] = incl;
        __syncthreads();
        int before = incl - hits, all = 0;
        for (int w = 0; w < PLACE_THREADS / 32; w++) {
            if (w < warp) before += warp_total[w];
            all += warp_total[w];
        }
        int at = base + placed + before;
        for (int i = i0; i < i1; i++) {
            const int c = chunk[i + (i >> 5)];
            if (c == e && e < experts) {
                pair_row[c0 + i] = at;
                row_token[at] = (c0 + i) / top;
                at++;
            } else if (e == 0 && c >= experts) {
                pair_row[c0 + i] = -1;
            }
        }
        placed += all;
    }
    const int mine = counts[e];
    const int padded = (mine + tile - 1) / tile * tile;
    for (int r = mine + threadIdx.x; r < padded; r += blockDim.x) row_token[base + r] = -1;
    for (int i = threadIdx.x; i < padded / tile; i += blockDim.x) tile_group[base / tile + i] = e;
    if (e == (int)gridDim.x - 1) {   // behind the last segment: tiles that are not in use, rows that are nobody's
        for (int i = (base + padded) / tile + threadIdx.x; i < max_tiles; i += blockDim.x) tile_group[i] = -1;
        for (long r = base + padded + threadIdx.x; r < (long)max_tiles * tile; r += blockDim.x) row_token[r] = -1;
        if (threadIdx.x == 0) tile_group[max_tiles] = (base + padded) / tile;   // how many tiles are in use: they come first
    }
}

// one block per token
template <typename TX>
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const TX* __restrict__ x, const int* __restrict__ pair_row,
                   const float* __restrict__ weight, int width, int top, int add) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float acc = add ? out[t * width + i] : 0.f;
        for (int k = 0; k < top; k++) {
            const int row = pair_row[t * top + k];
            const float v = row >= 0 ? y[(size_t)row * width + i] : to_float(x[t * width + i]);
            acc = fmaf(weight[t * top + k], v, acc);
        }
        out[t * width + i] = acc;
    }
}

// A step of few tokens in one block: the routing of every token, then the sorted rows, with what the three kernels above
// leave behind (chosen, weight, pair_row, row_token, tile_group).  A thread owns an expert and walks the pairs in order.
constexpr int SMALL_PAIRS = 1024, SMALL_THREADS = 256;

__global__ void __launch_bounds__(SMALL_THREADS)
moe_route_place_small_kernel(int* __restrict__ chosen, float* __restrict__ weight, int* __restrict__ pair_row, int* __restrict__ row_token,
                             int* __restrict__ tile_group, const float* __restrict__ logits, const float* __restrict__ correction,
                             const float* __restrict__ bias, int renorm, int tokens, int outputs, int top, int experts, int tile, int max_tiles) {
    extern __shared__ float smem[];   // [warps][2 * outputs] scores and choice scores, then [experts + 1] segment starts
    __shared__ int pairs_s[SMALL_PAIRS];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = SMALL_THREADS / 32;
    float* s = smem + (size_t)warp * 2 * outputs;
    float* c = s + outputs;
    int* start = reinterpret_cast<int*>(smem + (size_t)warps * 2 * outputs);
    for (int t = warp; t < tokens; t += warps) {
        const float* z = logits + (size_t)t * outputs;
        float m = -INFINITY;
        for (int i = lane; i < outputs; i += 32) m = fmaxf(m, z[i] + (bias ? bias[i] : 0.f));
        m = warp_max(m);
        float sum = 0.f;
        for (int i = lane; i < outputs; i += 32) { const float e = expf(z[i] + (bias ? bias[i] : 0.f) - m); s[i] = e; sum += e; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int i = lane; i < outputs; i += 32) {
            s[i] *= inv;
            c[i] = s[i] + (correction ? correction[i] : 0.f);
        }
        __syncwarp();
        for (int k = 0; k < top; k++) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int i = lane; i < outputs; i += 32)
                if (c[i] > best) { best = c[i]; at = i; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0) {
                chosen[(size_t)t * top + k] = at;
                weight[(size_t)t * top + k] = s[at];
                pairs_s[t * top + k] = at;
                c[at] = -INFINITY;
            }
            __syncwarp();
        }
        if (renorm && lane == 0) {
            float chosen_sum = 0.f;
            for (int k = 0; k < top; k++) chosen_sum += weight[(size_t)t * top + k];
            for (int k = 0; k < top; k++) weight[(size_t)t * top + k] /= chosen_sum;
        }
    }
    __syncthreads();
    const int pairs = tokens * top;
    for (int e = threadIdx.x; e < experts; e += SMALL_THREADS) {
        int n = 0;
        for (int i = 0; i < pairs; i++) n += pairs_s[i] == e;
        start[e + 1] = (n + tile - 1) / tile * tile;   // the segment's padded length for now
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        start[0] = 0;
        for (int e = 0; e < experts; e++) start[e + 1] += start[e];
        tile_group[max_tiles] = start[experts] / tile;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += SMALL_THREADS) {
        int at = start[e];
        for (int i = 0; i < pairs; i++)
            if (pairs_s[i] == e) { pair_row[i] = at; row_token[at] = i / top; at++; }
        for (; at < start[e + 1]; at++) row_token[at] = -1;
        for (int i = start[e] / tile; i < start[e + 1] / tile; i++) tile_group[i] = e;
    }
    for (int i = threadIdx.x; i < pairs; i += SMALL_THREADS)
        if (pairs_s[i] >= experts) pair_row[i] = -1;
    const int used = start[experts];
    for (int i = used / tile + threadIdx.x; i < max_tiles; i += SMALL_THREADS) tile_group[i] = -1;
    for (int r = used + threadIdx.x; r < max_tiles * tile; r += SMALL_THREADS) row_token[r] = -1;
}

// The mixture's last step and the norm behind the sublayer in one pass over a token's row:
//   v = (branch[t] if given) + sum_k weight[t, k] * (y[pair_row[t, k]] or x[t]);  residual[t] += v / rms(v) * gain;  rows[t] = residual[t] rounded
constexpr int COMBINE_MAX_TOP = 16;   // choices of a token whose rows and weights are held in shared memory

template <typename TX, typename TW, typename TH>
__global__ void __launch_bounds__(256)
moe_combine_norm_kernel(float* __restrict__ residual, TH* __restrict__ rows, const float* __restrict__ branch, const float* __restrict__ y,
                        const TX* __restrict__ x, const int* __restrict__ pair_row, const float* __restrict__ weight,
                        const TW* __restrict__ gain, int width, int top, float eps) {
    extern __shared__ float smem[];   // [width] the row, then 33 floats for the block sum
    __shared__ int row_s[COMBINE_MAX_TOP];
    __shared__ float weight_s[COMBINE_MAX_TOP];
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    // the token's rows and weights once, so that the loads of the loop below depend on nothing but their index
    const bool held = top <= COMBINE_MAX_TOP;
    if (held && threadIdx.x < top) {
        row_s[threadIdx.x] = pair_row[t * top + threadIdx.x];
        weight_s[threadIdx.x] = weight[t * top + threadIdx.x];
    }
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float acc = branch ? branch[t * width + i] : 0.f;
        const float own = to_float(x[t * width + i]);
        for (int k = 0; k < top; k++) {
            const int row = held ? row_s[k] : pair_row[t * top + k];
            const float v = row >= 0 ? y[(size_t)row * width + i] : own;
            acc = fmaf(held ? weight_s[k] : weight[t * top + k], v, acc);
        }
        smem[i] = acc;
        ss = fmaf(acc, acc, ss);
    }
    ss = block_sum(ss, smem + width);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = residual[t * width + i] + smem[i] * scale * to_float(gain[i]);
        residual[t * width + i] = v;
        if (rows) rows[t * width + i] = from_float<TH>(v);
    }
}

// xs[r] = x[row_token[r]] for the sorted rows (zeros for padding rows): the operand of a product whose tiles come by TMA
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(T* __restrict__ xs, const T* __restrict__ x, const int* __restrict__ row_token, int width, bool vec) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t r = blockIdx.x;
    const int t = row_token[r];
    constexpr int V = 16 / sizeof(T);
    if (vec) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(t < 0 ? 0 : t) * width);
        uint4* dst = reinterpret_cast<uint4*>(xs + r * width);
        for (int i = threadIdx.x; i < width / V; i += blockDim.x) dst[i] = t < 0 ? make_uint4(0, 0, 0, 0) : src[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) xs[r * width + i] = t < 0 ? from_float<T>(0.f) : x[(size_t)t * width + i];
    }
}

}  // namespace

HYMT2_API int hymt2_moe_gather(void* xs, const void* x, int dtype, const int* row_token, int rows, int width, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && width > 0 && row_token, "moe_gather: bad sizes");
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        const bool vec = width % (16 / sizeof(T)) == 0 && (uintptr_t)xs % 16 == 0 && (uintptr_t)x % 16 == 0;
        launch_pdl(moe_gather_kernel<T>, dim3(rows), dim3(128), 0, stream, (T*)xs, (const T*)x, row_token, width, vec);
    });
    return hymt2_check_launch("moe_gather");
}

HYMT2_API int hymt2_moe_route(int* chosen, float* weight, const float* logits, const float* correction, const float* bias, int renorm,
                              int tokens, int outputs, int top, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && outputs > 0 && top > 0 && top <= outputs, "moe_route: bad sizes tokens=%d outputs=%d top=%d", tokens, outputs, top);
    const size_t smem = (size_t)ROUTE_WARPS * 2 * outputs * sizeof(float);
    HYMT2_REQUIRE(smem <= 48 * 1024, "moe_route: %d router outputs are too many", outputs);
    launch_pdl(moe_route_kernel, dim3((tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, chosen, weight,
               logits, correction, bias, renorm, tokens, outputs, top);
    return hymt2_check_launch("moe_route");
}

// counts [experts] is scratch; row_token holds pairs + experts * (tile - 1) rows rounded up to whole tiles, tile_group one entry
// for each of those tiles (max_tiles) and one more, which receives the number of tiles in use (they are the first ones).
HYMT2_API int hymt2_moe_place(int* pair_row, int* row_token, int* tile_group, int* counts, const int* chosen, int tokens, int top,
                              int experts, int tile, int max_tiles, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && top > 0 && experts >= 0 && tile > 0, "moe_place: bad sizes");
    HYMT2_REQUIRE((long)tokens * top < (1L << 24), "moe_place: too many (token, choice) pairs");
    HYMT2_REQUIRE(experts == 0 || (long)max_tiles * tile >= (long)tokens * top + (long)experts * (tile - 1), "moe_place: too few tiles");
    const int pairs = tokens * top;
    const int blocks = experts > 0 ? experts : 1;
    launch_pdl(moe_count_kernel, dim3(blocks), dim3(PLACE_THREADS), 0, stream, counts, chosen, pairs, experts);
    launch_pdl(moe_place_kernel, dim3(blocks), dim3(PLACE_THREADS), 0, stream, pair_row, row_token, tile_group, (const int*)counts, chosen,
               pairs, top, experts, tile, max_tiles);
    return hymt2_check_launch("moe_place");
}

HYMT2_API int hymt2_moe_combine(float* out, const float* y, const void* x, int x_dtype, const int* pair_row, const float* weight,
                                int tokens, int width, int top, int add, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && width > 0 && top > 0, "moe_combine: bad sizes");
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, (launch_pdl(moe_combine_kernel<TX>, dim3(tokens), dim3(256), 0, stream, out, y, (const TX*)x, pair_row,
                                                  weight, width, top, add)));
    return hymt2_check_launch("moe_combine");
}

// moe_route and moe_place in one launch for a step of few tokens (tokens * top <= 1024, experts <= 4096).
HYMT2_API int hymt2_moe_route_place_small(int* chosen, float* weight, int* pair_row, int* row_token, int* tile_group, const float* logits,
                                          const float* correction, const float* bias, int renorm, int tokens, int outputs, int top, int experts,
                                          int tile, int max_tiles, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && outputs > 0 && top > 0 && top <= outputs && experts >= 0 && experts <= outputs && tile > 0, "moe_route_place_small: bad sizes");
    HYMT2_REQUIRE((long)tokens * top <= SMALL_PAIRS, "moe_route_place_small: %d pairs are too many", tokens * top);
    HYMT2_REQUIRE(experts == 0 || (long)max_tiles * tile >= (long)tokens * top + (long)experts * (tile - 1), "moe_route_place_small: too few tiles");
    const size_t smem = ((size_t)(SMALL_THREADS / 32) * 2 * outputs + experts + 1) * sizeof(float);
    HYMT2_REQUIRE(smem <= 40 * 1024, "moe_route_place_small: %d router outputs are too many", outputs);
    launch_pdl(moe_route_place_small_kernel, dim3(1), dim3(SMALL_THREADS), smem, stream, chosen, weight, pair_row, row_token, tile_group,
               logits, correction, bias, renorm, tokens, outputs, top, experts, tile, max_tiles);
    return hymt2_check_launch("moe_route_place");
}

// residual += norm(branch + the chosen experts' rows) with the norm's gain; rows (may be null) = the new residual rows in their type.
HYMT2_API int hymt2_moe_combine_norm(float* residual, void* rows, int rows_dtype, const float* branch, const float* y, const void* x,
                                     int x_dtype, const int* pair_row, const float* weight, const void* gain, int gain_dtype, int tokens,
                                     int width, int top, float eps, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && width > 0 && top > 0, "moe_combine_norm: bad sizes");
    const size_t smem = ((size_t)width + 33) * sizeof(float);
    HYMT2_REQUIRE(smem <= 48 * 1024, "moe_combine_norm: rows of %d entries are too wide", width);
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(rows_dtype, TH,
        (launch_pdl(moe_combine_norm_kernel<TX, TW, TH>, dim3(tokens), dim3(256), smem, stream, residual, (TH*)rows, branch, y, (const TX*)x,
                    pair_row, weight, (const TW*)gain, width, top, eps)))));
    return hymt2_check_launch("moe_combine_norm");
}
