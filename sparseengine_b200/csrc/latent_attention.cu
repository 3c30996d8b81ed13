// Attention over a cached latent: every position keeps one row `[c | k_rot]` of `rank + rot`
// elements (the normalised key/value latent and one rotated key part that all heads share) and
// no per-head keys or values.  Queries are taken into the latent's space before attention
// (`q_lat[h] = W_uk[h]^T q_plain[h]`, a matrix product outside this file), so that
//
//     score(i, j, h) = (q_lat[i, h] . c[j] + q_rot[i, h] . k_rot[j]) * scale
//     out_lat[i, h]  = sum_j softmax_j(score)(i, j, h) c[j]
//
// and the values' up-projection follows as one more product.  A query at position p sees keys
// max(0, p - window + 1) .. p (window 0: all keys).  With a sink the softmax's denominator also
// holds exp(sink[h]): a logit without key or value that is not scaled and counts once.
// Scores, weights and sums are 32-bit; the latent row is stored in the activation type.
//
// Kernels: the preparation of a step's tokens (RMS norms of the two latents in 32-bit, rotation
// of the shared key part, the page write), and attention with one block per (token, head) for any
// sizes; a tiled kernel for bfloat16 steps follows below.
#include "common.cuh"

namespace se {

#define SE_CODE_BAD_PAGE_LATENT_PREP 27
#define SE_CODE_BAD_PAGE_LATENT_ATTN 28

// One block per token.  proj row: [q latent (q_rank) | kv latent (rank) | shared key part (rot)].
//   cq_out[t]           = rmsnorm(q latent) * q_w                      (activation type)
//   page row [0, rank)  = rmsnorm(kv latent) * kv_w
//   page row [rank, ..) = the key part, its first `rotary_dim` dims rotated by the position
//                         (dim i pairs with i + rotary_dim/2; angle = position * inv_freq[i])
template <typename T>
__global__ void latent_prep_kernel(const T* proj, int proj_stride, const T* __restrict__ q_w, const T* __restrict__ kv_w,
                                   const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                   const int* __restrict__ token_seq, const int* __restrict__ seq_rows,
                                   const int* __restrict__ table, int table_stride, T* cache, T* cq_out, int q_rank,
                                   int rank, int rot, int rotary_dim, float eps, int page_size, int num_pages,
                                   int write_cache, int* error) {
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_float(row[i]); sq += v * v; }
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_float(row[q_rank + i]); sk += v * v; }
    const float inv_q = 1.0f / sqrtf(block_sum(sq, scratch) / (float)q_rank + eps);
    const float inv_k = 1.0f / sqrtf(block_sum(sk, scratch) / (float)rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
        cq_out[(size_t)t * q_rank + i] = from_float<T>(to_float(row[i]) * inv_q * to_float(q_w[i]));
    if (!write_cache) return;
    const int pos = positions[t];
    const int page = table[(size_t)seq_rows[token_seq[t]] * table_stride + pos / page_size];
    if (!page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_LATENT_PREP)) return;
    const int D = rank + rot;
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * D;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        dst[i] = from_float<T>(to_float(row[q_rank + i]) * inv_k * to_float(kv_w[i]));
    const T* kr = row + q_rank + rank;
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
        float v = to_float(kr[i]);
        if (i < rotary_dim) {
            const int j = i < half ? i : i - half;
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            const float u = to_float(kr[j]), w = to_float(kr[j + half]);
            v = i < half ? u * cs - w * sn : w * cs + u * sn;
        }
        dst[rank + i] = from_float<T>(v);
    }
}

constexpr int kLatWarps = 4;

// One block per (token, head); a warp takes every fourth key, lane l the dims l, l + 32, ...
// q_lat: float [heads, tokens, rank]; q: [tokens, heads * (d + rot)] in the activation type, of which
// the last `rot` of each head are the rotated part (rotated here); out: [heads, tokens, rank].
template <typename T, int NL>
__global__ void latent_attention_plain_kernel(const float* __restrict__ q_lat, const T* __restrict__ q, int d,
                                              const float* __restrict__ inv_freq, int rotary_dim,
                                              const T* __restrict__ cache, const int* __restrict__ table,
                                              int table_stride, const int* __restrict__ seq_rows,
                                              const int* __restrict__ token_seq, const int* __restrict__ positions,
                                              const float* __restrict__ sink, T* __restrict__ out, int tokens, int heads,
                                              int rank, int rot, int page_size, float scale, int window, int num_pages,
                                              int* __restrict__ error) {
    extern __shared__ float lat_smem[];          // [D] the query, then [warps][rank] partial sums
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int D = rank + rot;
    const int pos = positions[t];
    float* qs = lat_smem;
    float* sacc = lat_smem + D;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) qs[i] = q_lat[((size_t)h * tokens + t) * rank + i] * scale;
    const T* qr = q + ((size_t)t * heads + h) * (d + rot) + d;
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
        float v = to_float(qr[i]);
        if (i < rotary_dim) {
            const int j = i < half ? i : i - half;
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            const float u = to_float(qr[j]), w = to_float(qr[j + half]);
            v = i < half ? u * cs - w * sn : w * cs + u * sn;
        }
        qs[rank + i] = v * scale;
    }
    __syncthreads();
    float qreg[NL], acc[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        const int dim = lane + 32 * i;
        qreg[i] = dim < D ? qs[dim] : 0.f;
        acc[i] = 0.f;
    }
    const int* row_table = table + (size_t)seq_rows[token_seq[t]] * table_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= pos; j += kLatWarps) {
        const int page = row_table[j / page_size];
        if (!page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_LATENT_ATTN)) continue;
        const T* kp = cache + ((size_t)page * page_size + j % page_size) * D;
        float kv[NL];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            const int dim = lane + 32 * i;
            kv[i] = dim < D ? to_float(kp[dim]) : 0.f;
            s += qreg[i] * kv[i];
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < NL; ++i) acc[i] = acc[i] * corr + p * kv[i];      // dims beyond rank are dropped below
        m = m_new;
    }
    __shared__ float sm[kLatWarps], sl[kLatWarps];
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        const int dim = lane + 32 * i;
        if (dim < rank) sacc[warp * rank + dim] = acc[i];
    }
    __syncthreads();
    const float sk = sink != nullptr ? sink[h] : -INFINITY;
    float mt = sk;
#pragma unroll
    for (int w = 0; w < kLatWarps; ++w) mt = fmaxf(mt, sm[w]);
    float lt = sink != nullptr ? expf(sk - mt) : 0.f;
#pragma unroll
    for (int w = 0; w < kLatWarps; ++w) lt += sm[w] == -INFINITY ? 0.f : sl[w] * expf(sm[w] - mt);
    T* op = out + ((size_t)h * tokens + t) * rank;
    for (int dim = threadIdx.x; dim < rank; dim += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kLatWarps; ++w) o += sm[w] == -INFINITY ? 0.f : sacc[w * rank + dim] * expf(sm[w] - mt);
        op[dim] = from_float<T>(o / lt);
    }
}

}  // namespace se

extern "C" int se_latent_max_row() { return 32 * 20; }

extern "C" int se_latent_prep(const void* proj, int proj_stride, const void* q_w, const void* kv_w, const float* inv_freq,
                              const int* positions, const int* token_seq, const int* seq_rows, const int* table,
                              int table_stride, void* cache, void* cq_out, int tokens, int q_rank, int rank, int rot,
                              int rotary_dim, float eps, int page_size, int num_pages, int write_cache, int* error,
                              int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (q_rank <= 0 || rank <= 0 || rot < 0 || rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1) || page_size <= 0)
        return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::latent_prep_kernel<T><<<tokens, 128, 0, stream>>>((const T*)proj, proj_stride, (const T*)q_w, (const T*)kv_w,
            inv_freq, positions, token_seq, seq_rows, table, table_stride, (T*)cache, (T*)cq_out, q_rank, rank, rot,
            rotary_dim, eps, page_size, num_pages, write_cache, error));
    SE_LAUNCH_CHECK();
}

extern "C" int se_latent_attention_plain(const float* q_lat, const void* q, int d, const float* inv_freq, int rotary_dim,
                                         const void* cache, const int* table, int table_stride, const int* seq_rows,
                                         const int* token_seq, const int* positions, const float* sink, void* out,
                                         int tokens, int heads, int rank, int rot, int page_size, float scale, int window,
                                         int num_pages, int* error, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int D = rank + rot;
    if (rank <= 0 || rot < 0 || D > se_latent_max_row() || heads <= 0 || heads > 65535) return SE_ERR_UNSUPPORTED;
    if (rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1) || d < 0 || page_size <= 0) return SE_ERR_ARGUMENT;
    dim3 grid(tokens, heads);
    const size_t smem = (size_t)(D + se::kLatWarps * rank) * sizeof(float);
#define SE_LAT_LAUNCH(NL)                                                                                             \
    se::latent_attention_plain_kernel<T, NL><<<grid, 32 * se::kLatWarps, smem, stream>>>(                             \
        q_lat, (const T*)q, d, inv_freq, rotary_dim, (const T*)cache, table, table_stride, seq_rows, token_seq,        \
        positions, sink, (T*)out, tokens, heads, rank, rot, page_size, scale, window, num_pages, error)
    SE_DISPATCH_DTYPE(dtype, T, {
        if (D <= 128) SE_LAT_LAUNCH(4);
        else if (D <= 256) SE_LAT_LAUNCH(8);
        else SE_LAT_LAUNCH(20);
    });
#undef SE_LAT_LAUNCH
    SE_LAUNCH_CHECK();
}
