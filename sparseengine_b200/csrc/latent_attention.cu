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
// the last `rot` of each head are the rotated part (rotated here); out: [tokens, heads, rank].
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
    T* op = out + ((size_t)t * heads + h) * rank;
    for (int dim = threadIdx.x; dim < rank; dim += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kLatWarps; ++w) o += sm[w] == -INFINITY ? 0.f : sacc[w * rank + dim] * expf(sm[w] - mt);
        op[dim] = from_float<T>(o / lt);
    }
}

}  // namespace se

extern "C" int se_latent_max_row() { return 32 * 32; }

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
        else if (D <= 640) SE_LAT_LAUNCH(20);
        else SE_LAT_LAUNCH(32);
    });
#undef SE_LAT_LAUNCH
    SE_LAUNCH_CHECK();
}

// ---- the tiled kernel (bfloat16) ------------------------------------------------------------------
//
// All heads share a position's cached row, so the rows of a score tile are (token, head) pairs,
// token-major: a 64-row tile spans a few tokens and all their heads (or 64 heads of one token), and
// every key tile brought to shared memory serves all of them: a decode step reads a request's
// window once, not once per head.  Flash-attention loop on m16n8k16 tiles: the query tile stays in
// shared memory (A fragments by ldmatrix), each of four warps owns 16 rows, key tiles of 64 rows
// `[c | k_rot]` arrive by cp.async; S = Q K^T over all `D = rank + rot` dims, P V over the first
// `rank` dims of the same tile (the latent is the value).  Scores, softmax and sums are 32-bit; the
// sink joins a row's running maximum and sum before the first key.  Rows of the tile are stored
// with a pitch of DMAX elements, chunks of 16 bytes XOR-swizzled.
#include "mma_util.cuh"

namespace se {
namespace lat {

// Tiles of 64 rows; 64 keys for steps of single tokens, 32 keys for steps with prompt portions (fewer score and weight
// registers leave the compiler room to ask for the next fragments while the MMAs of these run: 198 -> 181 us over a
// 2,048-token prompt; three CTAs per SM at 168 registers did not pay, nor did a second set of score accumulators).
constexpr int kTileRows = 64;
constexpr int kWarps = 4;
constexpr int kThreads = 32 * kWarps;

using namespace se::mma;

// qfull[t, h, :] = [q_lat[h, t, :] | rotated part of q[t, h]] in bfloat16: the query rows as the tiled kernel reads them
__global__ void latent_q_pack_kernel(const float* __restrict__ q_lat, const __nv_bfloat16* __restrict__ q, int d,
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     const int* __restrict__ positions, __nv_bfloat16* __restrict__ qfull, int tokens,
                                     int heads, int rank, int rot) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int D = rank + rot;
    __nv_bfloat16* dst = qfull + ((size_t)t * heads + h) * D;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        dst[i] = __float2bfloat16_rn(q_lat[((size_t)h * tokens + t) * rank + i]);
    const __nv_bfloat16* qr = q + ((size_t)t * heads + h) * (d + rot) + d;
    const int half = rotary_dim / 2;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
        float v = __bfloat162float(qr[i]);
        if (i < rotary_dim) {
            const int j = i < half ? i : i - half;
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            const float u = __bfloat162float(qr[j]), w = __bfloat162float(qr[j + half]);
            v = i < half ? u * cs - w * sn : w * cs + u * sn;
        }
        dst[rank + i] = __float2bfloat16_rn(v);
    }
}

// D16T, RT: the row's 16-dim groups rounded up to a multiple of four (the tile's chunks between the row's end and that
// are zero-filled), and the same for the latent: loops of fixed length, no branch between the MMAs;
// output columns beyond the latent are computed and dropped.
template <int DMAX, int STAGES, int D16T, int RT, int TK, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
latent_attention_tiled_kernel(const __nv_bfloat16* __restrict__ qfull, const __nv_bfloat16* __restrict__ cache,
                              const int* __restrict__ table, int table_stride, const int* __restrict__ seq_rows,
                              const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                              const float* __restrict__ sink, __nv_bfloat16* __restrict__ out, int tokens, int heads,
                              int rank, int rot, int page_size, float scale, int window, int num_pages,
                              int* __restrict__ error, int splits, int tiles_per_split, float* __restrict__ part_o,
                              float* __restrict__ part_ml) {
    constexpr int kTileKeys = TK;
    constexpr int kTileBytes = kTileKeys * DMAX * 2;
    extern __shared__ __align__(128) uint8_t lat_tile_smem[];
    uint8_t* q_smem = lat_tile_smem;                     // [kTileRows][DMAX]
    uint8_t* k_smem = lat_tile_smem + kTileRows * DMAX * 2;   // [STAGES][kTileKeys][DMAX]
    const int D = rank + rot;
    const int chunks = D / 8;                            // 16-byte chunks of a row
    constexpr int kChunksT = 2 * D16T;                   // chunks the MMAs read; those beyond the row are zero
    const int r16 = rank / 16;

    const int entry = blockIdx.y;
    const int tok0 = cu_q[entry];
    const int q_len = cu_q[entry + 1] - tok0;
    const int total_rows = q_len * heads;
    const int row_base = (int)(gridDim.x - 1 - blockIdx.x) * kTileRows;     // the tiles with the most keys start first
    if (row_base >= total_rows) return;
    const int kv_end = kv_len[entry];
    const int q_start = kv_end - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;

    int pos[2], tok[2], head[2], lo[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row_base + warp * 16 + g + 8 * h;
        valid[h] = row < total_rows;
        const int r = valid[h] ? row : total_rows - 1;
        tok[h] = tok0 + r / heads;
        head[h] = r % heads;
        pos[h] = q_start + r / heads;
        lo[h] = window > 0 ? max(0, pos[h] - window + 1) : 0;
    }
    const int last_row = min(row_base + kTileRows, total_rows) - 1;
    const int max_pos = q_start + last_row / heads;
    const int first_pos = q_start + row_base / heads;
    const int k_lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int k_begin = (k_lo / kTileKeys) * kTileKeys;
    const int k_end = max_pos + 1;
    const int num_tiles = (k_end - k_begin + kTileKeys - 1) / kTileKeys;
    const int* row_table = table + (size_t)seq_rows[entry] * table_stride;
    // with several splits, CTA z takes the key tiles [t_begin, t_end) and leaves unnormalised sums
    // with their maximum for the merge kernel, which also brings the sink in
    const int t_begin = splits > 1 ? min(num_tiles, (int)blockIdx.z * tiles_per_split) : 0;
    const int t_end = splits > 1 ? min(num_tiles, t_begin + tiles_per_split) : num_tiles;
    const bool with_sink = sink != nullptr && splits == 1;

    // the query tile: rows are contiguous in qfull ([tokens, heads, D], token-major)
    {
        const __nv_bfloat16* src = qfull + ((size_t)tok0 * heads + row_base) * D;
        const int n_rows = min(kTileRows, total_rows - row_base);
        for (int x = threadIdx.x; x < kTileRows * kChunksT; x += kThreads) {
            const int r = x / kChunksT, c = x % kChunksT;
            const bool ok = r < n_rows && c < chunks;
            cp_async16(smem_u32(q_smem) + tile_off<DMAX>(r, c), src + (size_t)(ok ? r : 0) * D + (ok ? c : 0) * 8, ok);
        }
    }
    // A key row is copied by kThreads / kTileKeys neighbouring threads, 16 bytes each in turn: one block-table lookup
    // per thread and tile, and the threads of a row ask for adjacent bytes.
    constexpr int kPerRow = kThreads / kTileKeys;
    const int ld_row = threadIdx.x / kPerRow, ld_c0 = threadIdx.x % kPerRow;
    auto load_tile = [&](int tile, int stage) {
        uint8_t* kbase = k_smem + (size_t)stage * kTileBytes;
        const int j = k_begin + tile * kTileKeys + ld_row;
        // clamped into what every row of the tile may see: rows outside are zero-filled, never read (a
        // page behind the window may belong to another request by now)
        const int jj = min(max(j, k_lo), k_end - 1);
        const int page = row_table[jj / page_size];
        const bool row_ok = page_in_pool(page, num_pages, error, 29) && j < k_end && j >= k_lo;
        const __nv_bfloat16* src = cache + ((size_t)(row_ok ? page : 0) * page_size + jj % page_size) * D;
        const uint32_t dst = smem_u32(kbase);
#pragma unroll
        for (int c = ld_c0; c < kChunksT; c += kPerRow) {
            const bool ok = row_ok && c < chunks;
            cp_async16(dst + tile_off<DMAX>(ld_row, c), src + (ok ? c : 0) * 8, ok);
        }
    };
    for (int s = 0; s < STAGES - 1; ++s) {
        if (t_begin + s < t_end) load_tile(t_begin + s, s);
        cp_async_commit();                               // the first group also holds the query tile
    }

    float o[2 * RT][4];
#pragma unroll
    for (int i = 0; i < 2 * RT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // the sink: a logit of its own (not scaled) that joins the maximum and the sum; in units of the
    // raw scores it is sink / scale
    float m_run[2], l_run[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        m_run[h] = with_sink ? sink[head[h]] / scale : -INFINITY;
        l_run[h] = (with_sink && t4 == 0) ? 1.f : 0.f;           // the four lanes of a row add their sums at the end
    }
    const float scale_log2 = scale * 1.4426950408889634f;
    const int warp_last_row = min(row_base + warp * 16 + 15, total_rows - 1);
    const int warp_max_pos = q_start + warp_last_row / heads;
    const int warp_min_pos = q_start + min(row_base + warp * 16, total_rows - 1) / heads;
    const int warp_max_lo = window > 0 ? max(0, warp_max_pos - window + 1) : 0;
    const uint32_t qaddr = smem_u32(q_smem);

    for (int tile = t_begin; tile < t_end; ++tile) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (tile + STAGES - 1 < t_end) load_tile(tile + STAGES - 1, (tile - t_begin + STAGES - 1) % STAGES);
        cp_async_commit();

        const int key0 = k_begin + tile * kTileKeys;
        if (key0 > warp_max_pos || row_base + warp * 16 >= total_rows) continue;       // warp-uniform
        const uint32_t kaddr = smem_u32(k_smem + (size_t)((tile - t_begin) % STAGES) * kTileBytes);

        float s[kTileKeys / 8][4];
#pragma unroll
        for (int n = 0; n < kTileKeys / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int kk = 0; kk < D16T; ++kk) {
            uint32_t qa[4];
            ldmatrix_x4(qaddr + tile_off<DMAX>(warp * 16 + (mat & 1) * 8 + rr, 2 * kk + (mat >> 1)), qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
            for (int n2 = 0; n2 < kTileKeys / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kaddr + tile_off<DMAX>(n2 * 16 + (mat >> 1) * 8 + rr, 2 * kk + (mat & 1)), b0, b1, b2, b3);
                mma_bf16(s[2 * n2], qa, b0, b1);
                mma_bf16(s[2 * n2 + 1], qa, b2, b3);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
        // a tile that every row of the warp sees whole (most tiles of a long window) needs no mask
        if (key0 >= warp_max_lo && key0 + kTileKeys - 1 <= warp_min_pos) {
#pragma unroll
            for (int n = 0; n < kTileKeys / 8; ++n) {
                mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
            }
        } else {
#pragma unroll
            for (int n = 0; n < kTileKeys / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + n * 8 + 2 * t4 + (e & 1);
                    const int h = e >> 1;
                    if (j > pos[h] || j < lo[h]) s[n][e] = -INFINITY;
                    mx[h] = fmaxf(mx[h], s[n][e]);
                }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            corr[h] = exp2f((m_run[h] - m_use[h]) * scale_log2);
            m_run[h] = m_new;
        }
        float psum[2] = {0.f, 0.f};
        uint32_t pa[kTileKeys / 16][4];
#pragma unroll
        for (int n = 0; n < kTileKeys / 8; ++n) {
            const float p0 = exp2f((s[n][0] - m_use[0]) * scale_log2);
            const float p1 = exp2f((s[n][1] - m_use[0]) * scale_log2);
            const float p2 = exp2f((s[n][2] - m_use[1]) * scale_log2);
            const float p3 = exp2f((s[n][3] - m_use[1]) * scale_log2);
            psum[0] += p0 + p1;
            psum[1] += p2 + p3;
            pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + psum[h];
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {      // the running maxima mostly stand still
#pragma unroll
            for (int i = 0; i < 2 * RT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
        }
#pragma unroll
        for (int kk = 0; kk < kTileKeys / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < RT; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(kaddr + tile_off<DMAX>(kk * 16 + (mat & 1) * 8 + rr, 2 * n2 + (mat >> 1)), b0, b1, b2, b3);
                mma_bf16(o[2 * n2], pa[kk], b0, b1);
                mma_bf16(o[2 * n2 + 1], pa[kk], b2, b3);
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    if (splits > 1) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (!valid[h]) continue;
            const size_t at = ((size_t)tok[h] * heads + head[h]) * splits + blockIdx.z;
            if (t4 == 0) { part_ml[2 * at] = m_run[h]; part_ml[2 * at + 1] = l_run[h]; }
            float* dst = part_o + at * rank;
#pragma unroll
            for (int i = 0; i < 2 * RT; ++i)
                if (i < 2 * r16) *reinterpret_cast<float2*>(dst + i * 8 + 2 * t4) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!valid[h]) continue;
        const float inv = 1.f / l_run[h];
        __nv_bfloat16* dst = out + ((size_t)tok[h] * heads + head[h]) * rank;
#pragma unroll
        for (int i = 0; i < 2 * RT; ++i)
            if (i < 2 * r16)
                *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
}

// One block per (token, head): the splits' sums brought to one maximum, the sink added once.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const float* __restrict__ sink, __nv_bfloat16* __restrict__ out, int tokens,
                                              int heads, int rank, int splits, float scale) {
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t at = ((size_t)t * heads + h) * splits;
    const float scale_log2 = scale * 1.4426950408889634f;
    float mt = sink != nullptr ? sink[h] / scale : -INFINITY;
    for (int z = 0; z < splits; ++z) mt = fmaxf(mt, part_ml[2 * (at + z)]);
    float lt = sink != nullptr ? exp2f((sink[h] / scale - mt) * scale_log2) : 0.f;
    for (int z = 0; z < splits; ++z) {
        const float m = part_ml[2 * (at + z)];
        if (m != -INFINITY) lt += part_ml[2 * (at + z) + 1] * exp2f((m - mt) * scale_log2);
    }
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < splits; ++z) {
            const float m = part_ml[2 * (at + z)];
            if (m != -INFINITY) o += part_o[(at + z) * rank + c] * exp2f((m - mt) * scale_log2);
        }
        out[((size_t)t * heads + h) * rank + c] = __float2bfloat16_rn(o / lt);
    }
}

template <int DMAX, int STAGES, int D16T, int RT, int TK, int MINB>
static int launch_tiled(const void* qfull, const void* cache, const int* table, int table_stride, const int* seq_rows,
                        const int* cu_q, const int* kv_len, const float* sink, void* out, int tokens, int entries,
                        int max_q_len, int heads, int rank, int rot, int page_size, float scale, int window, int num_pages,
                        int* error, int splits, int tiles_per_split, float* part_o, float* part_ml, cudaStream_t stream) {
    const size_t smem = (size_t)(kTileRows + STAGES * TK) * DMAX * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_tiled_kernel<DMAX, STAGES, D16T, RT, TK, MINB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long row_tiles = ((long long)max_q_len * heads + kTileRows - 1) / kTileRows;
    if (row_tiles > 0x7fffffffLL || entries > 65535) return SE_ERR_UNSUPPORTED;
    dim3 grid((unsigned)row_tiles, entries, splits);
    latent_attention_tiled_kernel<DMAX, STAGES, D16T, RT, TK, MINB><<<grid, kThreads, smem, stream>>>(
        (const __nv_bfloat16*)qfull, (const __nv_bfloat16*)cache, table, table_stride, seq_rows, cu_q, kv_len, sink,
        (__nv_bfloat16*)out, tokens, heads, rank, rot, page_size, scale, window, num_pages, error, splits, tiles_per_split,
        part_o, part_ml);
    if (splits > 1)
        latent_attention_merge_kernel<<<dim3(tokens, heads), 64, 0, stream>>>(part_o, part_ml, sink, (__nv_bfloat16*)out,
                                                                             tokens, heads, rank, splits, scale);
    return (int)cudaGetLastError();
}

}  // namespace lat
}  // namespace se

// Sizes the tiled kernel takes: latent and rotated part in multiples of 16, a row of at most 256.
extern "C" int se_latent_attention_tiled_supported(int rank, int rot) {
    return rank > 0 && rot >= 0 && rank % 16 == 0 && rot % 16 == 0 && rank + rot <= 256;
}

extern "C" int se_latent_q_pack(const float* q_lat, const void* q, int d, const float* inv_freq, int rotary_dim,
                                const int* positions, void* qfull, int tokens, int heads, int rank, int rot,
                                cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1)) return SE_ERR_ARGUMENT;
    se::lat::latent_q_pack_kernel<<<dim3(tokens, heads), 64, 0, stream>>>(
        q_lat, (const __nv_bfloat16*)q, d, inv_freq, rotary_dim, positions, (__nv_bfloat16*)qfull, tokens, heads, rank, rot);
    SE_LAUNCH_CHECK();
}

// qfull: bfloat16 [tokens, heads, rank + rot]; out: bfloat16 [tokens, heads, rank]; cu_q: [entries + 1]
// token offsets; kv_len: [entries] keys of each request once this step's rows are written.
// splits > 1: the key tiles a row tile sees are dealt to `splits` CTAs, `tiles_per_split` tiles of 64 keys
// each (steps of few rows over long windows); part_o: float [tokens * heads * splits * rank], part_ml:
// float [tokens * heads * splits * 2].
extern "C" int se_latent_attention_tiled(const void* qfull, const void* cache, const int* table, int table_stride,
                                         const int* seq_rows, const int* cu_q, const int* kv_len, const float* sink,
                                         void* out, int tokens, int entries, int max_q_len, int heads, int rank, int rot,
                                         int page_size, float scale, int window, int num_pages, int* error, int splits,
                                         int tiles_per_split, float* part_o, float* part_ml, int tile_keys,
                                         cudaStream_t stream) {
    if (entries <= 0 || max_q_len <= 0) return 0;
    if (!se_latent_attention_tiled_supported(rank, rot) || heads <= 0 || heads > 65535) return SE_ERR_UNSUPPORTED;
    if (!(scale > 0.f) || page_size <= 0 || splits < 1 || splits > 65535) return SE_ERR_ARGUMENT;
    if (splits > 1 && (tiles_per_split < 1 || part_o == nullptr || part_ml == nullptr)) return SE_ERR_ARGUMENT;
    if (tile_keys != 64 && tile_keys != 32) return SE_ERR_ARGUMENT;
    const int d16t = (rank + rot + 63) / 64 * 4, rt = (rank + 63) / 64 * 4;
#define SE_LAT_ARGS qfull, cache, table, table_stride, seq_rows, cu_q, kv_len, sink, out, tokens, entries, max_q_len, heads, \
                    rank, rot, page_size, scale, window, num_pages, error, splits, tiles_per_split, part_o, part_ml, stream
#define SE_LAT_TILED(DMAX, STAGES, D16T, RT)                                                                          \
    if (d16t == D16T && rt == RT)                                                                                     \
        return tile_keys == 64 ? se::lat::launch_tiled<DMAX, STAGES, D16T, RT, 64, 1>(SE_LAT_ARGS)                     \
                               : se::lat::launch_tiled<DMAX, 3, D16T, RT, 32, 2>(SE_LAT_ARGS)
    SE_LAT_TILED(128, 3, 4, 4);
    SE_LAT_TILED(128, 3, 8, 4);
    SE_LAT_TILED(128, 3, 8, 8);
    SE_LAT_TILED(256, 2, 12, 4);
    SE_LAT_TILED(256, 2, 12, 8);
    SE_LAT_TILED(256, 2, 12, 12);
    SE_LAT_TILED(256, 2, 16, 4);
    SE_LAT_TILED(256, 2, 16, 8);
    SE_LAT_TILED(256, 2, 16, 12);
    SE_LAT_TILED(256, 2, 16, 16);
#undef SE_LAT_TILED
#undef SE_LAT_ARGS
    return SE_ERR_UNSUPPORTED;
}
