// Retention: linear attention with one fixed decay per head and no softmax or denominator.
//
//     S_t = decay[h] S_(t-1) + k_t v_t^T        (state [d, dv] per request and head, 32-bit)
//     o_t = S_t^T q_t
//
// q and k are rotated by their position on the first `rotary_dim` dims of each head (dim i pairs
// with i + rotary_dim/2, angle = position * inv_freq[i]); k is multiplied by `k_scale` after the
// rotation.  Each head's o is divided by its root mean square and multiplied by silu(gate).
// Rotation, scaling, state, sums and the norm are 32-bit; q, k, v and the gate come from the
// projection in the activation type.
//
// A step brings any mix of prompt portions and single tokens: entry s owns the tokens
// cu_q[s] .. cu_q[s+1]-1 and the state row seq_rows[s].
#include "common.cuh"

namespace se {

// q32, k32 [tokens, heads, d]: rotated (k also scaled), 32-bit.  One thread per (token, head, dim).
template <typename T>
__global__ void retention_prep_kernel(const T* proj, int proj_stride, int q_off, int k_off,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                      float* __restrict__ q32, float* __restrict__ k32, int tokens, int heads, int d,
                                      int rotary_dim, float k_scale) {
    const size_t n = (size_t)tokens * heads * d;
    const int half = rotary_dim / 2;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % d);
        const int h = (int)((idx / d) % heads);
        const int t = (int)(idx / ((size_t)d * heads));
        const T* qp = proj + (size_t)t * proj_stride + q_off + h * d;
        const T* kp = proj + (size_t)t * proj_stride + k_off + h * d;
        float qv = to_float(qp[i]), kv = to_float(kp[i]);
        if (i < rotary_dim) {
            const int j = i < half ? i : i - half;
            float sn, cs;
            sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
            const float qu = to_float(qp[j]), qw = to_float(qp[j + half]);
            const float ku = to_float(kp[j]), kw = to_float(kp[j + half]);
            qv = i < half ? qu * cs - qw * sn : qw * cs + qu * sn;
            kv = i < half ? ku * cs - kw * sn : kw * cs + ku * sn;
        }
        q32[idx] = qv;
        k32[idx] = kv * k_scale;
    }
}

constexpr int kRetWarps = 8;        // the state's rows are dealt to the warps: warp r holds rows r, r + 8, ...
constexpr int kRetTokens = 8;       // tokens staged at a time

// One block per (entry, head, 32 value columns).  Thread (warp r, lane c) keeps rows r + 8 n of column
// c in registers; a token's partial sums over a warp's rows meet in shared memory, eight tokens at
// a time.  Sums run in one fixed order whatever the batch or the portion.
template <typename T, int NPT>
__global__ void __launch_bounds__(32 * kRetWarps)
retention_scan_kernel(const float* __restrict__ q32, const float* __restrict__ k32, const T* proj, int proj_stride,
                      int v_off, const float* __restrict__ decay, float* state, long long state_stride,
                      const int* __restrict__ cu_q, const int* __restrict__ seq_rows, float* __restrict__ o, int heads,
                      int d, int dv) {
    extern __shared__ float ret_smem[];
    float* qs = ret_smem;                                   // [kRetTokens][d]
    float* ks = qs + kRetTokens * d;                        // [kRetTokens][d]
    float* vs = ks + kRetTokens * d;                        // [kRetTokens][32]
    float* red = vs + kRetTokens * 32;                      // [kRetTokens][kRetWarps][32]
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = c0 + lane;
    const bool col_ok = col < dv;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    if (t1 <= t0) return;
    const float g = decay[h];
    float* S = state + (size_t)seq_rows[s] * state_stride + (size_t)h * d * dv;
    float st[NPT];
#pragma unroll
    for (int n = 0; n < NPT; ++n) {
        const int i = warp + kRetWarps * n;
        st[n] = (i < d && col_ok) ? S[(size_t)i * dv + col] : 0.f;
    }
    for (int tb = t0; tb < t1; tb += kRetTokens) {
        const int nt = min(kRetTokens, t1 - tb);
        __syncthreads();                                    // the last round's sums have been read
        for (int x = threadIdx.x; x < nt * d; x += blockDim.x) {
            const int tt = x / d, i = x - tt * d;
            const size_t at = ((size_t)(tb + tt) * heads + h) * d + i;
            qs[tt * d + i] = q32[at];
            ks[tt * d + i] = k32[at];
        }
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int tt = x >> 5, c = x & 31;
            vs[x] = c0 + c < dv ? to_float(proj[(size_t)(tb + tt) * proj_stride + v_off + h * dv + c0 + c]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt * 32 + lane];
            float acc = 0.f;
#pragma unroll
            for (int n = 0; n < NPT; ++n) {
                const int i = warp + kRetWarps * n;
                if (i < d) {
                    st[n] = g * st[n] + ks[tt * d + i] * v;
                    acc += st[n] * qs[tt * d + i];
                }
            }
            red[(tt * kRetWarps + warp) * 32 + lane] = acc;
        }
        __syncthreads();
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int tt = x >> 5, c = x & 31;
            if (c0 + c < dv) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kRetWarps; ++w) sum += red[(tt * kRetWarps + w) * 32 + c];
                o[((size_t)(tb + tt) * heads + h) * dv + c0 + c] = sum;
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NPT; ++n) {
        const int i = warp + kRetWarps * n;
        if (i < d && col_ok) S[(size_t)i * dv + col] = st[n];
    }
}

// ---- prompt portions: the recurrence in chunks of 64 tokens ---------------------------------------
//
// With a fixed decay g the recurrence over a chunk of n tokens (local index t, s) has a closed form:
//
//     o_t   = g^(t+1) S_0^T q_t + sum_{s <= t} g^(t-s) (q_t . k_s) v_s
//     S_new = g^n S_0 + sum_s g^(n-1-s) k_s v_s^T
//
// which is three small matrix products per chunk instead of a chain of n dependent steps.  All of it
// is 32-bit FMA arithmetic (scores, decays and state enter the recurrence in 32-bit).  One block per
// (entry, head, 32 value columns): q and k of the chunk lie transposed in shared memory (`[dim][token]`, padded
// rows), the block's slice of the state stays in shared memory over all chunks.
constexpr int kChunk = 64;
constexpr int kChunkThreads = 256;

// a 4-byte asynchronous copy into shared memory: a chunk's q and k are all asked for before any of them is waited for
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// q and k of a chunk lie transposed, `[dim][token]`, rows padded to 68 floats: 16-byte reads along the tokens stay
// aligned, a walk along the dims is one add per step, and the transposing store spreads over 8 banks.
constexpr int kPitch = kChunk + 4;
__device__ __forceinline__ int swz(int i, int t) { return i * kPitch + t; }

template <typename T>
__global__ void __launch_bounds__(kChunkThreads, 2)
retention_chunk_kernel(const float* __restrict__ q32, const float* __restrict__ k32, const T* proj, int proj_stride,
                       int v_off, const float* __restrict__ decay, float* state, long long state_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ seq_rows, float* __restrict__ o, int heads,
                       int d, int dv, int max_seg, int seg_len, float* __restrict__ seg_state) {
    extern __shared__ __align__(16) float chunk_smem[];
    float* qs = chunk_smem;                      // [d][kPitch]
    float* ks = qs + d * kPitch;                 // [d][kPitch]
    float* vs = ks + d * kPitch;                 // [64][32]
    float* As = vs + kChunk * 32;                // [64 s][64 t]: g^(t-s) q_t . k_s for s <= t, else 0
    float* Ss = As + kChunk * kChunk;            // [d][32]
    float* gp = Ss + d * 32;                     // [65] powers of the decay
    // With segments (seg_state != nullptr) block x = entry * max_seg + segment walks `seg_len` tokens of its entry from
    // a zero state and leaves the state it ends with in seg_state; what the true state at the segment's start adds to
    // the outputs follows in retention_seg_fix_kernel.  Without, it walks the whole entry from the carried state.
    const int e = blockIdx.x / max_seg, sg = blockIdx.x - e * max_seg;
    const int h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, wg = threadIdx.x >> 5;
    const int t_first = seg_state != nullptr ? cu_q[e] + sg * seg_len : cu_q[e];
    const int t_last = seg_state != nullptr ? min(cu_q[e + 1], t_first + seg_len) : cu_q[e + 1];
    if (t_last <= t_first) return;
    const double g = (double)decay[h];
    for (int j = threadIdx.x; j <= kChunk; j += kChunkThreads) gp[j] = (float)pow(g, (double)j);
    float* S = seg_state != nullptr ? seg_state + (((size_t)e * max_seg + sg) * heads + h) * d * dv
                                    : state + (size_t)seq_rows[e] * state_stride + (size_t)h * d * dv;
    const bool col_ok = c0 + lane < dv;
    for (int x = threadIdx.x; x < d * 32; x += kChunkThreads)
        Ss[x] = (seg_state == nullptr && c0 + (x & 31) < dv) ? S[(size_t)(x >> 5) * dv + c0 + (x & 31)] : 0.f;

    const int ld_t0 = threadIdx.x / d, ld_i0 = threadIdx.x % d, ld_dt = kChunkThreads / d, ld_di = kChunkThreads % d;
    for (int tb = t_first; tb < t_last; tb += kChunk) {
        const int n = min(kChunk, t_last - tb);
        __syncthreads();                          // the chunk before is done with q, k, v and A; the state is up to date
        for (int x = threadIdx.x, t = ld_t0, i = ld_i0; x < kChunk * d; x += kChunkThreads) {      // (t, i) = (x / d, x % d)
            const size_t at = ((size_t)(tb + t) * heads + h) * d + i;
            if (t < n) {
                cp_async4(qs + swz(i, t), q32 + at);
                cp_async4(ks + swz(i, t), k32 + at);
            } else {
                qs[swz(i, t)] = 0.f;
                ks[swz(i, t)] = 0.f;
            }
            t += ld_dt;
            i += ld_di;
            if (i >= d) { i -= d; ++t; }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        for (int x = threadIdx.x; x < kChunk * 32; x += kChunkThreads) {
            const int t = x >> 5, c = x & 31;
            vs[x] = (t < n && c0 + c < dv) ? to_float(proj[(size_t)(tb + t) * proj_stride + v_off + h * dv + c0 + c]) : 0.f;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // scores of the chunk with their decays: a 4 x 4 tile per thread, tiles above the diagonal are zero
        {
            const int tt = (threadIdx.x >> 4) * 4, ss = (threadIdx.x & 15) * 4;
            float acc[4][4] = {};
            if (ss <= tt + 3) {
#pragma unroll 4
                for (int i = 0; i < d; ++i) {
                    const float4 qv = *reinterpret_cast<const float4*>(qs + swz(i, tt));
                    const float4 kv = *reinterpret_cast<const float4*>(ks + swz(i, ss));
                    const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                    for (int a = 0; a < 4; ++a)
#pragma unroll
                        for (int b = 0; b < 4; ++b) acc[a][b] += qa[a] * ka[b];
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float4 row;
                float* r = &row.x;
#pragma unroll
                for (int a = 0; a < 4; ++a) r[a] = (ss + b <= tt + a) ? acc[a][b] * gp[tt + a - ss - b] : 0.f;
                *reinterpret_cast<float4*>(As + (ss + b) * kChunk + tt) = row;
            }
        }
        float vreg[kChunk];                        // this lane's value column of the chunk
#pragma unroll
        for (int s_ = 0; s_ < kChunk; ++s_) vreg[s_] = vs[s_ * 32 + lane];
        __syncthreads();
        // outputs: warp wg takes tokens 8 wg .. 8 wg + 7, lane c the column
        {
            const int tg = wg * 8;
            float acc[8] = {}, acc2[8] = {};
#pragma unroll
            for (int s_ = 0; s_ < kChunk; ++s_) {
                const float4 a0 = *reinterpret_cast<const float4*>(As + s_ * kChunk + tg);
                const float4 a1 = *reinterpret_cast<const float4*>(As + s_ * kChunk + tg + 4);
                const float v = vreg[s_];
                acc[0] += a0.x * v; acc[1] += a0.y * v; acc[2] += a0.z * v; acc[3] += a0.w * v;
                acc[4] += a1.x * v; acc[5] += a1.y * v; acc[6] += a1.z * v; acc[7] += a1.w * v;
            }
#pragma unroll 4
            for (int i = 0; i < d; ++i) {
                const float4 q0 = *reinterpret_cast<const float4*>(qs + swz(i, tg));
                const float4 q1 = *reinterpret_cast<const float4*>(qs + swz(i, tg + 4));
                const float sv = Ss[i * 32 + lane];
                acc2[0] += q0.x * sv; acc2[1] += q0.y * sv; acc2[2] += q0.z * sv; acc2[3] += q0.w * sv;
                acc2[4] += q1.x * sv; acc2[5] += q1.y * sv; acc2[6] += q1.z * sv; acc2[7] += q1.w * sv;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = tg + j;
                if (t < n && col_ok) o[((size_t)(tb + t) * heads + h) * dv + c0 + lane] = acc[j] + gp[t + 1] * acc2[j];
            }
        }
        __syncthreads();                          // every read of the old state is done
        // the state after the chunk: warp wg takes rows wg, wg + 8, ...
#pragma unroll
        for (int s_ = 0; s_ < kChunk; ++s_) vreg[s_] = s_ < n ? vreg[s_] * gp[n - 1 - s_] : 0.f;
        const float gn = gp[n];
        for (int i = wg; i < d; i += kChunkThreads / 32) {
            float a = 0.f;
#pragma unroll
            for (int s4 = 0; s4 < kChunk; s4 += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(ks + swz(i, s4));
                a += kv.x * vreg[s4] + kv.y * vreg[s4 + 1] + kv.z * vreg[s4 + 2] + kv.w * vreg[s4 + 3];
            }
            Ss[i * 32 + lane] = gn * Ss[i * 32 + lane] + a;
        }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < d * 32; x += kChunkThreads)
        if (c0 + (x & 31) < dv) S[(size_t)(x >> 5) * dv + c0 + (x & 31)] = Ss[x];
}

// The segments of an entry joined: seg_state[e, j] holds what segment j alone leaves; it becomes the state at
// segment j's start, S_0 = the carried state, S_(j+1) = g^(len_j) S_j + (what segment j leaves), and the last one
// goes back to the entry's state row.  One thread per state element.
__global__ void retention_seg_join_kernel(float* __restrict__ seg_state, float* state, long long state_stride,
                                          const float* __restrict__ decay, const int* __restrict__ cu_q,
                                          const int* __restrict__ seq_rows, int heads, int d, int dv, int max_seg,
                                          int seg_len) {
    const int e = blockIdx.y, h = blockIdx.z;
    const int n = cu_q[e + 1] - cu_q[e];
    if (n <= 0) return;
    const int nseg = (n + seg_len - 1) / seg_len;
    const double g = (double)decay[h];
    const float g_full = (float)pow(g, (double)seg_len), g_last = (float)pow(g, (double)(n - (nseg - 1) * seg_len));
    float* S = state + (size_t)seq_rows[e] * state_stride + (size_t)h * d * dv;
    for (int x = blockIdx.x * blockDim.x + threadIdx.x; x < d * dv; x += gridDim.x * blockDim.x) {
        float cur = S[x];
        for (int j = 0; j < nseg; ++j) {
            float* p = seg_state + (((size_t)e * max_seg + j) * heads + h) * d * dv + x;
            const float left = *p;
            *p = cur;
            cur = (j == nseg - 1 ? g_last : g_full) * cur + left;
        }
        S[x] = cur;
    }
}

// o_t += g^(t' + 1) S_start^T q_t for the tokens of a segment (t' counts from the segment's start): what the state at
// the segment's start adds to outputs that were computed from a zero state.  Same tiles as the chunked kernel.
__global__ void __launch_bounds__(kChunkThreads, 2)
retention_seg_fix_kernel(const float* __restrict__ q32, const float* __restrict__ seg_state, const float* __restrict__ decay,
                         const int* __restrict__ cu_q, float* __restrict__ o, int heads, int d, int dv, int max_seg,
                         int seg_len) {
    extern __shared__ __align__(16) float fix_smem[];
    float* qs = fix_smem;                        // [d][kPitch]
    float* Ss = qs + d * kPitch;                 // [d][32]
    float* gp = Ss + d * 32;                     // [seg_len + 1]
    const int e = blockIdx.x / max_seg, sg = blockIdx.x - e * max_seg;
    const int h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, wg = threadIdx.x >> 5;
    const int t_first = cu_q[e] + sg * seg_len, t_last = min(cu_q[e + 1], t_first + seg_len);
    if (t_last <= t_first) return;
    const double g = (double)decay[h];
    for (int j = threadIdx.x; j <= seg_len; j += kChunkThreads) gp[j] = (float)pow(g, (double)j);
    const float* S = seg_state + (((size_t)e * max_seg + sg) * heads + h) * d * dv;
    for (int x = threadIdx.x; x < d * 32; x += kChunkThreads) Ss[x] = (c0 + (x & 31) < dv) ? S[(size_t)(x >> 5) * dv + c0 + (x & 31)] : 0.f;
    const bool col_ok = c0 + lane < dv;
    for (int tb = t_first; tb < t_last; tb += kChunk) {
        const int n = min(kChunk, t_last - tb);
        __syncthreads();
        for (int x = threadIdx.x, t = threadIdx.x / d, i = threadIdx.x % d; x < kChunk * d; x += kChunkThreads) {
            if (t < n) cp_async4(qs + swz(i, t), q32 + ((size_t)(tb + t) * heads + h) * d + i);
            else qs[swz(i, t)] = 0.f;
            t += kChunkThreads / d;
            i += kChunkThreads % d;
            if (i >= d) { i -= d; ++t; }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const int tg = wg * 8;
        float acc2[8] = {};
#pragma unroll 4
        for (int i = 0; i < d; ++i) {
            const float4 q0 = *reinterpret_cast<const float4*>(qs + swz(i, tg));
            const float4 q1 = *reinterpret_cast<const float4*>(qs + swz(i, tg + 4));
            const float sv = Ss[i * 32 + lane];
            acc2[0] += q0.x * sv; acc2[1] += q0.y * sv; acc2[2] += q0.z * sv; acc2[3] += q0.w * sv;
            acc2[4] += q1.x * sv; acc2[5] += q1.y * sv; acc2[6] += q1.z * sv; acc2[7] += q1.w * sv;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int t = tg + j;
            if (t < n && col_ok) o[((size_t)(tb + t) * heads + h) * dv + c0 + lane] += gp[tb - t_first + t + 1] * acc2[j];
        }
    }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * silu(gate[t, h, :]); a warp per (token, head).
template <typename T>
__global__ void retention_out_kernel(const float* __restrict__ o, const T* proj, int proj_stride, int g_off,
                                     T* __restrict__ out, int rows, int heads, int dv, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int t = r / heads, h = r - t * heads;
    const float* op = o + (size_t)r * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += op[i] * op[i];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    const T* gp = proj + (size_t)t * proj_stride + g_off + h * dv;
    for (int i = lane; i < dv; i += 32) {
        const float gv = to_float(gp[i]);
        out[(size_t)r * dv + i] = from_float<T>(op[i] * inv * (gv / (1.f + expf(-gv))));
    }
}

}  // namespace se

extern "C" int se_retention_max_head_dim() { return se::kRetWarps * 32; }

extern "C" int se_retention_prep(const void* proj, int proj_stride, int q_off, int k_off, const float* inv_freq,
                                 const int* positions, float* q32, float* k32, int tokens, int heads, int d,
                                 int rotary_dim, float k_scale, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || d <= 0 || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1)) return SE_ERR_ARGUMENT;
    const long long n = (long long)tokens * heads * d;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    SE_DISPATCH_DTYPE(dtype, T,
        se::retention_prep_kernel<T><<<blocks, 256, 0, stream>>>((const T*)proj, proj_stride, q_off, k_off, inv_freq,
                                                                  positions, q32, k32, tokens, heads, d, rotary_dim, k_scale));
    SE_LAUNCH_CHECK();
}

extern "C" int se_retention_scan(const float* q32, const float* k32, const void* proj, int proj_stride, int v_off,
                                 const float* decay, float* state, long long state_stride, const int* cu_q,
                                 const int* seq_rows, float* o, int entries, int heads, int d, int dv, int dtype,
                                 cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (d <= 0 || d > se_retention_max_head_dim() || dv <= 0 || heads <= 0 || heads > 65535 || (dv + 31) / 32 > 65535)
        return SE_ERR_UNSUPPORTED;
    dim3 grid(entries, heads, (dv + 31) / 32);
    const size_t smem = (size_t)(2 * se::kRetTokens * d + se::kRetTokens * 32 + se::kRetTokens * se::kRetWarps * 32) * sizeof(float);
#define SE_RET_LAUNCH(NPT)                                                                                          \
    se::retention_scan_kernel<T, NPT><<<grid, 32 * se::kRetWarps, smem, stream>>>(                                  \
        q32, k32, (const T*)proj, proj_stride, v_off, decay, state, state_stride, cu_q, seq_rows, o, heads, d, dv)
    SE_DISPATCH_DTYPE(dtype, T, {
        if (d <= 8 * se::kRetWarps) SE_RET_LAUNCH(8);
        else if (d <= 16 * se::kRetWarps) SE_RET_LAUNCH(16);
        else SE_RET_LAUNCH(32);
    });
#undef SE_RET_LAUNCH
    SE_LAUNCH_CHECK();
}

// The same recurrence in chunks of 64 tokens (closed form per chunk): for steps with prompt portions.
extern "C" int se_retention_chunk_supported(int d) { return d > 0 && d <= 256; }

extern "C" int se_retention_chunk(const float* q32, const float* k32, const void* proj, int proj_stride, int v_off,
                                  const float* decay, float* state, long long state_stride, const int* cu_q,
                                  const int* seq_rows, float* o, int entries, int heads, int d, int dv, int max_seg,
                                  int seg_len, float* seg_state, int dtype, cudaStream_t stream) {
    // max_seg > 1: the entries' tokens in segments of seg_len (a multiple of 64) that run side by side, joined by
    // the decay's powers (three launches); seg_state: float [entries, max_seg, heads, d, dv].
    if (entries <= 0) return 0;
    if (!se_retention_chunk_supported(d) || dv <= 0 || heads <= 0 || heads > 65535 || (dv + 31) / 32 > 65535)
        return SE_ERR_UNSUPPORTED;
    if (max_seg < 1 || (max_seg > 1 && (seg_state == nullptr || seg_len <= 0 || seg_len % se::kChunk || seg_len > 8192)))
        return SE_ERR_ARGUMENT;
    if ((long long)entries * max_seg > 0x7fffffffLL || entries > 65535) return SE_ERR_UNSUPPORTED;
    const bool segments = max_seg > 1;
    dim3 grid(entries * max_seg, heads, (dv + 31) / 32);
    const size_t smem = (size_t)(2 * d * se::kPitch + se::kChunk * 32 + se::kChunk * se::kChunk + d * 32 + se::kChunk + 4) * sizeof(float);
    SE_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e = cudaFuncSetAttribute(se::retention_chunk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // the largest shared-memory carve-out, so that two blocks share an SM where their tiles allow it
        e = cudaFuncSetAttribute(se::retention_chunk_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        se::retention_chunk_kernel<T><<<grid, se::kChunkThreads, smem, stream>>>(
            q32, k32, (const T*)proj, proj_stride, v_off, decay, state, state_stride, cu_q, seq_rows, o, heads, d, dv,
            max_seg, segments ? seg_len : 0, segments ? seg_state : nullptr);
    });
    if (segments) {
        const int per = d * dv;
        se::retention_seg_join_kernel<<<dim3((per + 255) / 256 < 64 ? (per + 255) / 256 : 64, entries, heads), 256, 0, stream>>>(
            seg_state, state, state_stride, decay, cu_q, seq_rows, heads, d, dv, max_seg, seg_len);
        const size_t fix_smem = (size_t)(d * se::kPitch + d * 32 + seg_len + 4) * sizeof(float);
        cudaError_t e = cudaFuncSetAttribute(se::retention_seg_fix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fix_smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(se::retention_seg_fix_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        se::retention_seg_fix_kernel<<<grid, se::kChunkThreads, fix_smem, stream>>>(q32, seg_state, decay, cu_q, o, heads, d, dv,
                                                                                  max_seg, seg_len);
    }
    SE_LAUNCH_CHECK();
}

extern "C" int se_retention_out(const float* o, const void* proj, int proj_stride, int g_off, void* out, int tokens,
                                int heads, int dv, float eps, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int rows = tokens * heads;
    SE_DISPATCH_DTYPE(dtype, T,
        se::retention_out_kernel<T><<<(rows + 7) / 8, 256, 0, stream>>>(o, (const T*)proj, proj_stride, g_off, (T*)out,
                                                                         rows, heads, dv, eps));
    SE_LAUNCH_CHECK();
}
