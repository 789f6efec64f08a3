// Low-rank (latent) key/value attention: what happens between the fused projection and the attention itself.
//
// The projection of a token holds, side by side, the queries of all heads (per head `dim` entries that meet the
// keys made from the latent vector, then `rot` entries that meet the rotated key part) and the compressed row
// (`rank` entries of the latent vector, then `rot` entries of the one rotated key part that all heads share).
// This kernel, one block per token, all arithmetic in float32:
//   * divides the latent vector by its root mean square (eps inside the root), multiplies it by its gain and
//     writes it to the token's row of the cache, entries [0, rank);
//   * rotates the shared key part by the token's position and writes it behind it, entries [rank, rank + rot);
//   * rotates the `rot` part of every head's query and writes it to q_out[t, h, rank .. rank + rot): the place
//     behind the head's `rank` entries, which the product with the key up-projection fills.
// Rotation: of the first `rot_dims` entries, (2i, 2i+1) are a pair that turns by angle = position * inv_freq[i]
// (a float32 product); cosine and sine are multiplied by `amplitude`; entries from rot_dims on pass unchanged.
// Cache plane: [block][token in block][rank + rot]; block_table[slot * table_stride + pos / block_tokens] names
// the block.  A token of a padding row (slot < 0) writes its query part and nothing else.
#include "common.cuh"

namespace {

struct LatentPrepParams {
    const void* proj;     // [T, ldp]
    void* q_out;          // [T, heads * (rank + rot)], or null: the rotated query parts go back into proj, in place
    void* rows_out;       // [T, rank + rot] or null: the compressed rows once more, side by side for all tokens
    void* cache;          // plane base, or null: nothing is written (a run that reads another run's cache)
    const int* block_table;
    const int* token_seq;
    const int* token_pos;
    const int* slot_ids;
    const float* gain;      // [rank]
    const float* inv_freq;  // [rot_dims / 2]
    long ldp;
    int q_cols;             // where the compressed row starts inside a projection row (= heads * (dim + rot))
    int table_stride, block_tokens, heads, dim, rot, rank, rot_dims;
    float eps, amplitude;
};

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(LatentPrepParams p) {
    extern __shared__ float smem[];   // [rot_dims / 2][2] cosine, sine; then 33 floats for the sum
    float* cs = smem;
    float* scratch = smem + p.rot_dims;
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = p.token_pos[t];
    const int slot = p.slot_ids[p.token_seq[t]];
    const T* row = (const T*)p.proj + (size_t)t * p.ldp;
    const int half = p.rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = (float)pos * p.inv_freq[i];
        float sn, c;
        sincosf(angle, &sn, &c);
        cs[2 * i] = c * p.amplitude;
        cs[2 * i + 1] = sn * p.amplitude;
    }
    // the latent vector's sum of squares (block_sum synchronises, which also publishes cs)
    const T* lat = row + p.q_cols;
    float ss = 0.f;
    if (p.cache || p.rows_out)      // (a projection without a compressed row of its own is never read behind its queries)
        for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
            const float v = to_float(lat[i]);
            ss = fmaf(v, v, ss);
        }
    ss = block_sum(ss, scratch);
    const int dl = p.rank + p.rot;
    T* dst = nullptr;    // the token's cache row
    if (p.cache && slot >= 0) {
        const int block = p.block_table[(size_t)slot * p.table_stride + pos / p.block_tokens];
        dst = (T*)p.cache + ((size_t)block * p.block_tokens + (pos % p.block_tokens)) * dl;
    }
    T* dst2 = p.rows_out ? (T*)p.rows_out + (size_t)t * dl : nullptr;
    if (dst || dst2) {
        const float scale = 1.0f / sqrtf(ss / (float)p.rank + p.eps);
        for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
            const T v = from_float<T>(to_float(lat[i]) * scale * p.gain[i]);
            if (dst) dst[i] = v;
            if (dst2) dst2[i] = v;
        }
        const T* kr = lat + p.rank;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float a = to_float(kr[2 * i]), b = to_float(kr[2 * i + 1]);
            const T v0 = from_float<T>(a * cs[2 * i] - b * cs[2 * i + 1]), v1 = from_float<T>(b * cs[2 * i] + a * cs[2 * i + 1]);
            if (dst) { dst[p.rank + 2 * i] = v0; dst[p.rank + 2 * i + 1] = v1; }
            if (dst2) { dst2[p.rank + 2 * i] = v0; dst2[p.rank + 2 * i + 1] = v1; }
        }
        for (int i = p.rot_dims + threadIdx.x; i < p.rot; i += blockDim.x) {
            if (dst) dst[p.rank + i] = kr[i];
            if (dst2) dst2[p.rank + i] = kr[i];
        }
    }
    // the heads' rotated query parts
    const int per_head = half + (p.rot - p.rot_dims);
    for (int item = threadIdx.x; item < p.heads * per_head; item += blockDim.x) {
        const int h = item / per_head, i = item - h * per_head;
        const T* q = row + (size_t)h * (p.dim + p.rot) + p.dim;
        T* o = p.q_out ? (T*)p.q_out + (size_t)t * p.heads * dl + (size_t)h * dl + p.rank : const_cast<T*>(q);
        if (i < half) {
            const float a = to_float(q[2 * i]), b = to_float(q[2 * i + 1]);
            o[2 * i] = from_float<T>(a * cs[2 * i] - b * cs[2 * i + 1]);
            o[2 * i + 1] = from_float<T>(b * cs[2 * i] + a * cs[2 * i + 1]);
        } else {
            const int x = p.rot_dims + (i - half);
            o[x] = q[x];
        }
    }
}

}  // namespace

HYMT2_API int hymt2_latent_prep(const void* proj, long ldp, int q_cols, void* q_out, void* rows_out, void* cache, int dtype,
                                const int* block_table, int table_stride, int block_tokens, const int* token_seq,
                                const int* token_pos, const int* slot_ids, const float* gain, const float* inv_freq,
                                int rot_dims, float amplitude, float eps, int tokens, int heads, int dim, int rot, int rank,
                                cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && heads > 0 && dim >= 0 && rot >= 0 && rank > 0, "latent_prep: bad sizes");
    HYMT2_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot, "latent_prep: %d rotated entries of %d", rot_dims, rot);
    HYMT2_REQUIRE(rot_dims == 0 || inv_freq != nullptr, "latent_prep: no frequencies");
    LatentPrepParams p;
    p.proj = proj; p.q_out = q_out; p.rows_out = rows_out; p.cache = cache; p.block_table = block_table; p.token_seq = token_seq;
    p.token_pos = token_pos; p.slot_ids = slot_ids; p.gain = gain; p.inv_freq = inv_freq; p.ldp = ldp; p.q_cols = q_cols;
    p.table_stride = table_stride; p.block_tokens = block_tokens; p.heads = heads; p.dim = dim; p.rot = rot; p.rank = rank;
    p.rot_dims = rot_dims; p.eps = eps; p.amplitude = amplitude;
    const size_t smem = sizeof(float) * ((size_t)rot_dims + 33);
    HYMT2_DISPATCH_DTYPE(dtype, T, launch_pdl(latent_prep_kernel<T>, dim3(tokens), dim3(128), smem, stream, p));
    return hymt2_check_launch("latent_prep");
}
