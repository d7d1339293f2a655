// Kernels for attention through low-rank latents, and the small pieces of the designs that use it.
//
// A position leaves ONE row behind for all heads: [c | r], c the normalised low-rank row (kv_rank channels) from
// which every head's keys and values are up-projections, r a small rotated key part that all heads share. The pages
// hold these rows and nothing else. Attention runs in the latent space: a head's query is carried through its key
// up-projection once (q_lat = [W_uk_h^T q_plain | rotate(q_rot)]), so that score = q_lat . [c | r], the context is
// the weighted sum of the c rows, and the head's value up-projection is applied to that sum:
//
//   layer_norm        (x - mean) / sqrt(var + eps) * w per row, float in, compute dtype out, optional row gather
//   latent_prepare    per token: rmsnorm of the query latent -> cq; rmsnorm of the kv latent and the rotation of the
//                     shared key part -> the token's row in its page
//   latent_query      per (token, head): q_lat from the up-projected query
//   latent_attention  paged attention of H query heads over the one row per position; values are the first kv_rank
//                     channels of the key row; window optional; keys in chunks of 128 aligned to absolute positions,
//                     chunk results merged in ascending order (in the CTA, or by latent_attention_merge when a
//                     decode step spreads a token's chunks over CTAs; the arithmetic is the same, so the bits are);
//                     for single tokens in bfloat16 a tensor-core form: a token's heads are the rows of mma.sync
//                     tiles over chunks of 64 keys held in shared memory (latent_attention_tc, merge_flat)
//   latent_output     per (token, head): W_uv_h applied to the latent context, times sigmoid(gate) and a constant
//   route_sigmoid     router with sigmoid scores, a correction that only the choice sees, weights not renormalised
//   scaled_relu_sq    hidden layer of ungated experts: relu(x)^2 times the token's weight for the expert
//   scale_softcap     logits <- cap * tanh(logits * scale / cap), in place
//
// Storage float or bfloat16, arithmetic float. Every sum is taken in an order that depends on sizes and absolute
// positions only, never on the batch.
#include "common.cuh"

IB_DEFINE_LAST_ERROR()

#define IB_LAUNCH(kernel, grid, block, smem, ...)                                                              \
    do {                                                                                                       \
        const int rc_ = ib::launch(#kernel, kernel, dim3(grid), dim3(block), size_t(smem), stream, 1u, __VA_ARGS__); \
        if (rc_) return rc_;                                                                                   \
    } while (0)

namespace {

using bf16 = __nv_bfloat16;

inline unsigned blocks_for(int64_t n, int threads) { return unsigned((n + threads - 1) / threads); }

__device__ __forceinline__ float sigmoid_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------------------
// Layer norm with a weight and no bias. One CTA per output row; the row waits in shared memory between the passes
// (mean, mean of squared deviations, result).
constexpr int LN_THREADS = 256;

template <typename TOut>
__global__ void __launch_bounds__(LN_THREADS)
layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int64_t hidden,
                  const int* __restrict__ rows, TOut* __restrict__ out) {
    ib::pdl_wait();
    extern __shared__ float ln_row[];
    __shared__ float red[32];
    const int64_t r = blockIdx.x;
    const float* src = x + (rows ? int64_t(rows[r]) : r) * hidden;
    float s = 0.0f;
    for (int64_t i = threadIdx.x; i < hidden; i += LN_THREADS) {
        const float v = src[i];
        ln_row[i] = v;
        s += v;
    }
    const float mean = ib::block_sum(s, red) / float(hidden);
    float q = 0.0f;
    for (int64_t i = threadIdx.x; i < hidden; i += LN_THREADS) {
        const float d = ln_row[i] - mean;
        q = fmaf(d, d, q);
    }
    const float inv = 1.0f / sqrtf(ib::block_sum(q, red) / float(hidden) + eps);
    for (int64_t i = threadIdx.x; i < hidden; i += LN_THREADS)
        out[r * hidden + i] = ib::from_f32<TOut>((ln_row[i] - mean) * inv * w[i]);
}

// ------------------------------------------------------------------------------------------------
// The two latents of a token, from the float rows of the down-projections [.. | query latent | .. | kv latent, shared
// key part | ..]. Query latent: divided by its root mean square, times wq -> cq. Kv latent likewise with wkv -> the
// first kv_rank channels of the token's row in its page; the shared key part is rotated by the token's position
// (tables [positions][n_rot / 2]; layout 0: channel 2i turns with 2i + 1, layout 1: channel i with i + n_rot / 2;
// channels from n_rot on pass) and follows. Either half may be absent (q_rank 0; write 0).
constexpr int LP_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(LP_THREADS)
latent_prepare_kernel(const float* __restrict__ rows, int64_t ld, int q_col, int q_rank, int kv_col, int kv_rank, int rot_dim,
                      const float* __restrict__ wq, const float* __restrict__ wkv, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int layout, int n_rot, const int* __restrict__ positions,
                      const int* __restrict__ token_seg, const int* __restrict__ block_table, int64_t max_blocks,
                      T* __restrict__ cq, T* __restrict__ cache, int page_size, int64_t n_pages, int write, int* status) {
    ib::pdl_wait();
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x;
    const float* src = rows + t * ld;
    if (q_rank > 0) {
        float s = 0.0f;
        for (int i = tid; i < q_rank; i += LP_THREADS) {
            const float v = src[q_col + i];
            s = fmaf(v, v, s);
        }
        const float inv = 1.0f / sqrtf(ib::block_sum(s, red) / float(q_rank) + eps);
        for (int i = tid; i < q_rank; i += LP_THREADS) cq[t * q_rank + i] = ib::from_f32<T>(src[q_col + i] * inv * wq[i]);
    }
    if (!write) return;
    float s = 0.0f;
    for (int i = tid; i < kv_rank; i += LP_THREADS) {
        const float v = src[kv_col + i];
        s = fmaf(v, v, s);
    }
    const float inv = 1.0f / sqrtf(ib::block_sum(s, red) / float(kv_rank) + eps);
    const int pos = positions[t];
    const int page = block_table[int64_t(token_seg[t]) * max_blocks + pos / page_size];
    if (page < 0 || page >= n_pages) {
        if (status && tid == 0) atomicExch(status, 2);
        return;
    }
    T* dst = cache + (int64_t(page) * page_size + pos % page_size) * (kv_rank + rot_dim);
    for (int i = tid; i < kv_rank; i += LP_THREADS) dst[i] = ib::from_f32<T>(src[kv_col + i] * inv * wkv[i]);
    const float* r = src + kv_col + kv_rank;
    T* rd = dst + kv_rank;
    const int half = n_rot / 2;
    for (int i = tid; i < half; i += LP_THREADS) {
        const int a = layout == 0 ? 2 * i : i, b = layout == 0 ? 2 * i + 1 : i + half;
        const float c = cos_t[int64_t(pos) * half + i], sn = sin_t[int64_t(pos) * half + i];
        const float u = r[a], v = r[b];
        rd[a] = ib::from_f32<T>(u * c - v * sn);
        rd[b] = ib::from_f32<T>(v * c + u * sn);
    }
    for (int i = n_rot + tid; i < rot_dim; i += LP_THREADS) rd[i] = ib::from_f32<T>(r[i]);
}

// ------------------------------------------------------------------------------------------------
// Products of a step's rows with one small matrix per head: out[t, h, n] = sum_k a[t, h, k] * B[h][k][n], B row-major
// with n contiguous. One CTA of 256 threads per (HP_TOK tokens, head, tile of HP_CL * C columns), C = 16 bytes of T per
// thread: narrow tiles, so that a step of few tokens still spreads a head's matrix over many CTAs. A thread owns C
// neighbouring columns of every token and every 64th k (k = slice, slice + 64, ...), so a matrix row is read once, by
// 16-byte loads, for all HP_TOK tokens; the 64 slice sums of a column are added in a fixed order (the eight slices of
// a warp by shuffles, then the eight warps in order through shared memory). The order of a sum depends on k
// alone: a token's result does not depend on which other tokens share its CTA. Leaves the eight warps' partial sums
// in `red` [8][HP_TOK][HP_CL * C] behind a barrier.
// With `seg_start` the CTAs serve the tokens of one-token segments only: rows of longer segments are neither read nor
// written (their attention runs elsewhere).
constexpr int HP_TOK = 8, HP_THREADS = 256, HP_CL = 4, HP_KS = HP_THREADS / HP_CL, HP_WARPS = HP_THREADS / 32;

template <typename T>
struct HpCols { static constexpr int v = 16 / int(sizeof(T)); };

template <typename T>
__device__ __forceinline__ void load_cols(const T* p, float (&x)[HpCols<T>::v]);
template <>
__device__ __forceinline__ void load_cols<float>(const float* p, float (&x)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
}
template <>
__device__ __forceinline__ void load_cols<bf16>(const bf16* p, float (&x)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

template <typename T>
__device__ __forceinline__ void head_product_tile(const float* __restrict__ a_s, const T* __restrict__ B, int K, int N, int n0,
                                                  bool vec, float* __restrict__ red) {
    constexpr int C = HpCols<T>::v, NT = HP_CL * C;
    const int tid = threadIdx.x, cl = tid % HP_CL, ks = tid / HP_CL, warp = tid >> 5, lane = tid & 31;
    const int nb = n0 + cl * C;
    float acc[HP_TOK][C];
#pragma unroll
    for (int tt = 0; tt < HP_TOK; tt++)
#pragma unroll
        for (int c = 0; c < C; c++) acc[tt][c] = 0.0f;
    if (nb < N) {
#pragma unroll 4
        for (int k = ks; k < K; k += HP_KS) {
            float w[C];
            const T* src = B + int64_t(k) * N + nb;
            if (vec) {
                load_cols<T>(src, w);
            } else {
#pragma unroll
                for (int c = 0; c < C; c++) w[c] = nb + c < N ? ib::to_f32(src[c]) : 0.0f;
            }
#pragma unroll
            for (int tt = 0; tt < HP_TOK; tt++) {
                const float a = a_s[tt * K + k];
#pragma unroll
                for (int c = 0; c < C; c++) acc[tt][c] = fmaf(a, w[c], acc[tt][c]);
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < HP_TOK; tt++)
#pragma unroll
        for (int c = 0; c < C; c++) {
#pragma unroll
            for (int off = HP_CL; off < 32; off *= 2) acc[tt][c] += __shfl_xor_sync(0xffffffffu, acc[tt][c], off);
        }
    if (lane < HP_CL) {
#pragma unroll
        for (int tt = 0; tt < HP_TOK; tt++)
#pragma unroll
            for (int c = 0; c < C; c++) red[(warp * HP_TOK + tt) * NT + cl * C + c] = acc[tt][c];
    }
    __syncthreads();
}

// bit tt of the result: token t0 + tt exists and (without seg_start) counts, or lies in a one-token segment
__device__ __forceinline__ unsigned tokens_served(int64_t t0, int nt, const int* __restrict__ token_seg, const int* __restrict__ seg_start) {
    unsigned mask = 0;
    for (int tt = 0; tt < nt; tt++) {
        bool on = true;
        if (seg_start) {
            const int sg = token_seg[t0 + tt];
            on = seg_start[sg + 1] - seg_start[sg] == 1;
        }
        mask |= on ? 1u << tt : 0u;
    }
    return mask;
}

// ------------------------------------------------------------------------------------------------
// Queries in the latent space. q [T][H][d + dr] (a head's unrotated channels, then its rotated ones); w_uk [H][d][R]
// (the key up-projection as checkpoints store it, [H * d, R]); out [T][H][R + dr]:
//   out[t, h, r] = sum_e q[t, h, e] * w_uk[h, e, r],  out[t, h, R:] = rotate(q[t, h, d:], position).
template <typename T>
__global__ void __launch_bounds__(HP_THREADS)
latent_query_kernel(const T* __restrict__ q, const T* __restrict__ w_uk, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int layout, int n_rot, const int* __restrict__ positions,
                    T* __restrict__ out, int64_t n_tokens, int n_heads, int d, int dr, int R, int vec,
                    const int* __restrict__ token_seg, const int* __restrict__ seg_start) {
    ib::pdl_wait();
    constexpr int NT = HP_CL * HpCols<T>::v;
    extern __shared__ __align__(16) float hp_sm[];
    float* a_s = hp_sm;                               // [HP_TOK][d]
    float* red = a_s + HP_TOK * d;                    // [HP_WARPS][HP_TOK][NT]
    const int64_t t0 = int64_t(blockIdx.x) * HP_TOK;
    const int h = blockIdx.y, tid = threadIdx.x;
    const int nt = int(min(int64_t(HP_TOK), n_tokens - t0));
    const unsigned served = tokens_served(t0, nt, token_seg, seg_start);
    if (!served) return;
    for (int i = tid; i < HP_TOK * d; i += HP_THREADS) {
        const int tt = i / d, e = i - tt * d;
        a_s[i] = (served >> tt & 1u) ? ib::to_f32(q[((t0 + tt) * n_heads + h) * (d + dr) + e]) : 0.0f;
    }
    __syncthreads();
    const int n0 = blockIdx.z * NT;
    head_product_tile<T>(a_s, w_uk + int64_t(h) * d * R, d, R, n0, vec != 0, red);
    for (int i = tid; i < HP_TOK * NT; i += HP_THREADS) {
        const int tt = i / NT, n = n0 + (i - tt * NT);
        if (!(served >> tt & 1u) || n >= R) continue;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < HP_WARPS; w++) s += red[(w * HP_TOK + tt) * NT + (n - n0)];
        out[((t0 + tt) * n_heads + h) * (R + dr) + n] = ib::from_f32<T>(s);
    }
    if (blockIdx.z == 0) {
        const int half = n_rot / 2;
        for (int i = tid; i < nt * half; i += HP_THREADS) {
            const int tt = i / half, j = i - tt * half;
            if (!(served >> tt & 1u)) continue;
            const int64_t t = t0 + tt;
            const int pos = positions[t];
            const int a = layout == 0 ? 2 * j : j, b = layout == 0 ? 2 * j + 1 : j + half;
            const float c = cos_t[int64_t(pos) * half + j], sn = sin_t[int64_t(pos) * half + j];
            const T* src = q + (t * n_heads + h) * (d + dr) + d;
            T* dst = out + (t * n_heads + h) * (R + dr) + R;
            const float u = ib::to_f32(src[a]), v = ib::to_f32(src[b]);
            dst[a] = ib::from_f32<T>(u * c - v * sn);
            dst[b] = ib::from_f32<T>(v * c + u * sn);
        }
        const int rest = dr - n_rot;
        for (int i = tid; i < nt * rest; i += HP_THREADS) {
            const int tt = i / rest, j = n_rot + (i - tt * rest);
            if (!(served >> tt & 1u)) continue;
            const int64_t t = t0 + tt;
            out[(t * n_heads + h) * (R + dr) + R + j] = q[(t * n_heads + h) * (d + dr) + d + j];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Attention over the latent rows. Keys are taken in chunks of KC positions aligned to absolute multiples of KC. A
// chunk gives, per head, its own maximum m, the sum l of exp(score - m) and the unnormalised context o; chunks are
// merged in ascending order by merge_state / merge_value below, whoever merges.
constexpr int KC = 128;
constexpr int VT = 32;                 // value rows staged at a time
constexpr int GMAX = 8;                // query heads that share a CTA's key rows

__device__ __forceinline__ void merge_state(float& M, float& L, float m, float l, float& a, float& b) {
    const float Mn = fmaxf(M, m);
    a = M == -INFINITY ? 0.0f : expf(M - Mn);
    b = m == -INFINITY ? 0.0f : expf(m - Mn);
    L = fmaf(L, a, l * b);
    M = Mn;
}
__device__ __forceinline__ float merge_value(float O, float a, float o, float b) { return fmaf(O, a, o * b); }

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float (&x)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

// GB: heads of a CTA rounded up to 1, 2, 4 or 8; NC: channel passes of a thread (dv <= NC * KC).
// With `seg_start`, tokens of segments longer than one token are left out (their attention runs elsewhere).
// n_splits 1: the CTA walks all chunks of its token and writes the context. n_splits > 1 (steps of single tokens):
// CTA z takes chunk z of its token and leaves (m, l, o) in `parts` [token][head][split][2 + dv].
template <typename T, int GB, int NC>
__global__ void __launch_bounds__(KC)
latent_attention_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_table,
                        int64_t max_blocks, const int* __restrict__ token_seg, const int* __restrict__ positions,
                        T* __restrict__ out, float* __restrict__ parts, int n_heads, int group, int dk, int dv, int page_size,
                        int window, float scale, int64_t n_pages, int n_splits, int vec, int vec_v, int* status,
                        const int* __restrict__ seg_start) {
    ib::pdl_wait();
    const int64_t t = blockIdx.x;
    const int g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (seg_start) {                                     // tokens of one-token segments only
        const int sg = token_seg[t];
        if (seg_start[sg + 1] - seg_start[sg] != 1) return;
    }
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int c_lo = lo / KC, c_hi = pos / KC;
    int c_first = c_lo, c_last = c_hi;
    if (n_splits > 1) {
        c_first = c_last = c_lo + int(blockIdx.z);
        if (c_first > c_hi) return;
    }
    const int h0 = g * group, ng = min(group, n_heads - h0);
    extern __shared__ __align__(16) float la_sm[];
    const int dq = (dk + 3) & ~3;
    float* qs = la_sm;                                   // [GB][dq]
    float* sc = qs + GB * dq;                            // [GB][KC] scores, then probabilities
    float* ml = sc + GB * KC;                            // [GB][2]
    int64_t* rowoff = reinterpret_cast<int64_t*>(ml + 2 * GMAX);   // [KC]
    T* vt = reinterpret_cast<T*>(rowoff + KC);           // [VT][dv]
    for (int i = tid; i < GB * dq; i += KC) {
        const int gq = i / dq, e = i - gq * dq;
        qs[i] = (gq < ng && e < dk) ? ib::to_f32(q[(t * n_heads + h0 + gq) * dk + e]) : 0.0f;
    }
    __syncthreads();
    const int* table = block_table + int64_t(token_seg[t]) * max_blocks;
    float M[GB], L[GB], O[GB][NC];
#pragma unroll
    for (int gq = 0; gq < GB; gq++) {
        M[gq] = -INFINITY;
        L[gq] = 0.0f;
#pragma unroll
        for (int c = 0; c < NC; c++) O[gq][c] = 0.0f;
    }
    for (int ch = c_first; ch <= c_last; ch++) {
        const int base = ch * KC, key = base + tid;
        const bool valid = key >= lo && key <= pos;
        float acc[GB];
#pragma unroll
        for (int gq = 0; gq < GB; gq++) acc[gq] = 0.0f;
        bool have = false;
        rowoff[tid] = 0;
        if (valid) {
            const int page = table[key / page_size];
            if (page < 0 || page >= n_pages) {
                if (status) atomicExch(status, 3);
            } else {
                have = true;
                const int64_t row = int64_t(page) * page_size + key % page_size;
                rowoff[tid] = row;
                const T* kr = cache + row * dk;
                if (vec) {
                    for (int e0 = 0; e0 < dk; e0 += 32) {
                        float kv[4][8];
#pragma unroll
                        for (int b4 = 0; b4 < 4; b4++)
                            if (e0 + 8 * b4 < dk) load8<T>(kr + e0 + 8 * b4, kv[b4]);
#pragma unroll
                        for (int b4 = 0; b4 < 4; b4++) {
                            const int e = e0 + 8 * b4;
                            if (e < dk) {
#pragma unroll
                                for (int gq = 0; gq < GB; gq++) {
                                    const float4 a = *reinterpret_cast<const float4*>(qs + gq * dq + e);
                                    const float4 b = *reinterpret_cast<const float4*>(qs + gq * dq + e + 4);
                                    float x = acc[gq];
                                    x = fmaf(a.x, kv[b4][0], x); x = fmaf(a.y, kv[b4][1], x); x = fmaf(a.z, kv[b4][2], x); x = fmaf(a.w, kv[b4][3], x);
                                    x = fmaf(b.x, kv[b4][4], x); x = fmaf(b.y, kv[b4][5], x); x = fmaf(b.z, kv[b4][6], x); x = fmaf(b.w, kv[b4][7], x);
                                    acc[gq] = x;
                                }
                            }
                        }
                    }
                } else {
                    for (int e = 0; e < dk; e++) {
                        const float kv = ib::to_f32(kr[e]);
#pragma unroll
                        for (int gq = 0; gq < GB; gq++) acc[gq] = fmaf(qs[gq * dq + e], kv, acc[gq]);
                    }
                }
            }
        }
#pragma unroll
        for (int gq = 0; gq < GB; gq++) sc[gq * KC + tid] = have ? acc[gq] * scale : -INFINITY;
        __syncthreads();
        for (int gq = warp; gq < GB; gq += KC / 32) {
            float* row = sc + gq * KC;
            float m = -INFINITY;
            for (int j = lane; j < KC; j += 32) m = fmaxf(m, row[j]);
            m = ib::warp_max(m);
            float l = 0.0f;
            for (int j = lane; j < KC; j += 32) {
                const float pv = row[j] > -INFINITY ? expf(row[j] - m) : 0.0f;
                row[j] = pv;
                l += pv;
            }
            l = ib::warp_sum(l);
            if (lane == 0) { ml[2 * gq] = m; ml[2 * gq + 1] = l; }
        }
        __syncthreads();
        const int j0 = max(lo, base) - base, j1 = min(pos, base + KC - 1) - base;
        float o[GB][NC];
#pragma unroll
        for (int gq = 0; gq < GB; gq++)
#pragma unroll
            for (int c = 0; c < NC; c++) o[gq][c] = 0.0f;
        for (int js = j0; js <= j1; js += VT) {
            const int nj = min(VT, j1 - js + 1);
            __syncthreads();                                 // the last staged rows have been read
            if (vec_v) {
                constexpr int PER = 16 / int(sizeof(T));
                const int per_row = dv / PER;
                for (int i = tid; i < nj * per_row; i += KC) {
                    const int jj = i / per_row, e = (i - jj * per_row) * PER;
                    *reinterpret_cast<uint4*>(vt + jj * dv + e) = *reinterpret_cast<const uint4*>(cache + rowoff[js + jj] * dk + e);
                }
            } else {
                for (int i = tid; i < nj * dv; i += KC) {
                    const int jj = i / dv, e = i - jj * dv;
                    vt[jj * dv + e] = cache[rowoff[js + jj] * dk + e];
                }
            }
            __syncthreads();
#pragma unroll 2
            for (int jj = 0; jj < nj; jj++) {
                float vv[NC];
#pragma unroll
                for (int c = 0; c < NC; c++) vv[c] = tid + c * KC < dv ? ib::to_f32(vt[jj * dv + tid + c * KC]) : 0.0f;
#pragma unroll
                for (int gq = 0; gq < GB; gq++) {
                    const float pj = sc[gq * KC + js + jj];
#pragma unroll
                    for (int c = 0; c < NC; c++) o[gq][c] = fmaf(pj, vv[c], o[gq][c]);
                }
            }
        }
#pragma unroll
        for (int gq = 0; gq < GB; gq++) {
            float a, b;
            merge_state(M[gq], L[gq], ml[2 * gq], ml[2 * gq + 1], a, b);
#pragma unroll
            for (int c = 0; c < NC; c++) O[gq][c] = merge_value(O[gq][c], a, o[gq][c], b);
        }
        __syncthreads();                                     // sc, ml and rowoff are free for the next chunk
    }
    if (n_splits > 1) {
#pragma unroll
        for (int gq = 0; gq < GB; gq++) {
            if (gq < ng) {
                float* dst = parts + ((t * n_heads + h0 + gq) * n_splits + blockIdx.z) * int64_t(dv + 2);
                if (tid == 0) { dst[0] = M[gq]; dst[1] = L[gq]; }
#pragma unroll
                for (int c = 0; c < NC; c++)
                    if (tid + c * KC < dv) dst[2 + tid + c * KC] = O[gq][c];
            }
        }
        return;
    }
#pragma unroll
    for (int gq = 0; gq < GB; gq++) {
        if (gq < ng) {
            const float inv = L[gq] > 0.0f ? 1.0f / L[gq] : 0.0f;
#pragma unroll
            for (int c = 0; c < NC; c++)
                if (tid + c * KC < dv) out[(t * n_heads + h0 + gq) * dv + tid + c * KC] = ib::from_f32<T>(O[gq][c] * inv);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// The same attention for single tokens in bfloat16 on the tensor cores (mma.sync m16n8k16): the heads of a token are
// the rows of the tile. One CTA of four warps per (token, group of 16 heads, chunk of TC_KC keys aligned to absolute
// multiples of TC_KC); it always leaves (m, l, o) in `parts`, and the merge kernel follows. The chunk's rows come
// into shared memory by 16-byte asynchronous copies (dk a multiple of 8), rows outside [lo, pos] as zeros; they serve
// as keys (all dk channels) and as values (the first dv). Warp w computes the scores of keys 16 w .. 16 w + 15, the
// maxima and sums cross the warps through shared memory, the probabilities are left there as two bfloat16 terms
// (p = hi + lo), and warp w then sums channels [16 NV w, 16 NV (w + 1)) over all keys.
constexpr int TC_KC = 64, TC_THREADS = 128, TC_HEADS = 16, TC_PS = TC_KC + 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void split_bf16(float x, bf16& hi, bf16& lo) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

// row stride of the chunk's rows in shared memory: dk rounded up to 16, plus 8 (an odd number of 16-byte units)
__host__ __device__ inline int tc_row_stride(int dk) { return ((dk + 15) & ~15) + 8; }

template <int NV>
__global__ void __launch_bounds__(TC_THREADS)
latent_attention_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, const int* __restrict__ block_table,
                           int64_t max_blocks, const int* __restrict__ token_seg, const int* __restrict__ positions,
                           float* __restrict__ parts, int n_heads, int dk, int dv, int page_size, int window, float scale,
                           int64_t n_pages, int n_splits, int* status, const int* __restrict__ seg_start) {
    ib::pdl_wait();
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (seg_start) {
        const int sg = token_seg[t];
        if (seg_start[sg + 1] - seg_start[sg] != 1) return;
    }
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int ch = lo / TC_KC + int(blockIdx.z);
    if (ch > pos / TC_KC) return;
    const int h0 = blockIdx.y * TC_HEADS, ng = min(TC_HEADS, n_heads - h0);
    const int RS = tc_row_stride(dk), dkp = RS - 8;
    extern __shared__ __align__(16) unsigned char tc_sm[];
    bf16* Qs = reinterpret_cast<bf16*>(tc_sm);               // [16][RS]
    bf16* Ks = Qs + TC_HEADS * RS;                           // [TC_KC][RS] (+ slack for the last warp's channel tiles)
    bf16* Ph = Ks + TC_KC * RS + 64 * NV;                 // [16][TC_PS]
    bf16* Pl = Ph + TC_HEADS * TC_PS;                        // [16][TC_PS]
    float* red = reinterpret_cast<float*>(Pl + TC_HEADS * TC_PS);   // [2][4][16] maxima, sums
    const int* table = block_table + int64_t(token_seg[t]) * max_blocks;
    const int cpr = dkp / 8, real = dk / 8, base = ch * TC_KC;
    {
        // two threads per key row: one page lookup per thread, then every other 16-byte piece of the row
        static_assert(TC_THREADS == 2 * TC_KC, "two threads per key row");
        const int row = tid >> 1, key = base + row;
        const bf16* src = nullptr;
        if (key >= lo && key <= pos) {
            const int page = table[key / page_size];
            if (page < 0 || page >= n_pages) {
                if (status) atomicExch(status, 3);
            } else {
                src = cache + (int64_t(page) * page_size + key % page_size) * dk;
            }
        }
        const uint32_t dst = smem_u32(Ks + row * RS);
        for (int c = tid & 1; c < cpr; c += 2) {
            const bool on = src && c < real;
            cp_async16(dst + c * 16, on ? src + c * 8 : cache, on ? 16 : 0);
        }
    }
    {
        // eight threads per head row of the queries
        static_assert(TC_THREADS == 8 * TC_HEADS, "eight threads per query row");
        const int row = tid >> 3;
        const bf16* src = row < ng ? q + (t * n_heads + h0 + row) * dk : nullptr;
        const uint32_t dst = smem_u32(Qs + row * RS);
        for (int c = tid & 7; c < cpr; c += 8) {
            const bool on = src && c < real;
            cp_async16(dst + c * 16, on ? src + c * 8 : q, on ? 16 : 0);
        }
    }
    cp_async_wait_all();
    __syncthreads();
    // scores of this warp's 16 keys for all 16 heads
    float sc[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
    for (int ks = 0; ks < dkp / 16; ks++) {
        uint32_t a[4], b[4];
        ldsm4(smem_u32(Qs + (lane & 15) * RS + ks * 16 + (lane >> 4) * 8), a);
        ldsm4(smem_u32(Ks + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * RS + ks * 16 + ((lane >> 3) & 1) * 8), b);
        mma16816(sc[0], a, b[0], b[1]);
        mma16816(sc[1], a, b[2], b[3]);
    }
    // rows lane / 4 and lane / 4 + 8 (heads), columns: keys base + 16 warp + 8 nt + 2 (lane % 4) + {0, 1}
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int key = base + warp * 16 + nt * 8 + (lane & 3) * 2 + (c & 1);
            const float v = (key >= lo && key <= pos) ? sc[nt][c] * scale : -INFINITY;
            sc[nt][c] = v;
            if (c < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
        }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const int ra = lane >> 2, rb = ra + 8;
    if ((lane & 3) == 0) { red[warp * 16 + ra] = mx_a; red[warp * 16 + rb] = mx_b; }
    __syncthreads();
    float m_a = -INFINITY, m_b = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; w++) { m_a = fmaxf(m_a, red[w * 16 + ra]); m_b = fmaxf(m_b, red[w * 16 + rb]); }
    const float ba = m_a == -INFINITY ? 0.0f : m_a, bb = m_b == -INFINITY ? 0.0f : m_b;
    float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const float pv = sc[nt][c] > -INFINITY ? expf(sc[nt][c] - (c < 2 ? ba : bb)) : 0.0f;
            if (c < 2) sum_a += pv; else sum_b += pv;
            const int col = warp * 16 + nt * 8 + (lane & 3) * 2 + (c & 1), row = c < 2 ? ra : rb;
            bf16 hi, lw;
            split_bf16(pv, hi, lw);
            Ph[row * TC_PS + col] = hi;
            Pl[row * TC_PS + col] = lw;
        }
    }
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
    if ((lane & 3) == 0) { red[64 + warp * 16 + ra] = sum_a; red[64 + warp * 16 + rb] = sum_b; }
    __syncthreads();
    // O = P V for this warp's channels
    float o[2 * NV][4];
#pragma unroll
    for (int i = 0; i < 2 * NV; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const int c0 = warp * NV * 16;
    if (c0 < dv) {
#pragma unroll
        for (int kk = 0; kk < TC_KC / 16; kk++) {
            uint32_t ph[4], pl[4];
            ldsm4(smem_u32(Ph + (lane & 15) * TC_PS + kk * 16 + (lane >> 4) * 8), ph);
            ldsm4(smem_u32(Pl + (lane & 15) * TC_PS + kk * 16 + (lane >> 4) * 8), pl);
#pragma unroll
            for (int np = 0; np < NV; np++) {
                uint32_t b[4];
                ldsm4_t(smem_u32(Ks + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + c0 + np * 16 + (lane >> 4) * 8), b);
                mma16816(o[2 * np], ph, b[0], b[1]);
                mma16816(o[2 * np + 1], ph, b[2], b[3]);
                mma16816(o[2 * np], pl, b[0], b[1]);
                mma16816(o[2 * np + 1], pl, b[2], b[3]);
            }
        }
    }
#pragma unroll
    for (int half_i = 0; half_i < 2; half_i++) {
        const int row = half_i ? rb : ra;
        if (row >= ng) continue;
        float* dst = parts + ((t * n_heads + h0 + row) * n_splits + blockIdx.z) * int64_t(dv + 2);
        if (warp == 0 && (lane & 3) == 0) {
            float l = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; w++) l += red[64 + w * 16 + row];
            dst[0] = half_i ? m_b : m_a;
            dst[1] = l;
        }
#pragma unroll
        for (int i = 0; i < 2 * NV; i++) {
            const int col = c0 + i * 8 + (lane & 3) * 2;
            if (col + 1 < dv && !(dv & 1)) {                // an even dv keeps every pair on an 8-byte boundary
                *reinterpret_cast<float2*>(dst + 2 + col) = make_float2(o[i][2 * half_i], o[i][2 * half_i + 1]);
            } else {
                if (col < dv) dst[2 + col] = o[i][2 * half_i];
                if (col + 1 < dv) dst[2 + col + 1] = o[i][2 * half_i + 1];
            }
        }
    }
}

// One CTA per (token, head), one thread per channel: the chunks' parts merged in ascending order, then the division.
// The chunks' maxima and sums wait in shared memory; every thread walks the same chain over them, and its own loads
// of the parts' channels do not depend on the chain, so they are in flight together.
constexpr int MG_THREADS = 128, MG_STAGE = 256;

template <typename T>
__global__ void __launch_bounds__(MG_THREADS)
latent_attention_merge_kernel(const float* __restrict__ parts, const int* __restrict__ positions, T* __restrict__ out,
                              int n_heads, int dv, int window, int n_splits, int chunk, const int* __restrict__ token_seg,
                              const int* __restrict__ seg_start) {
    ib::pdl_wait();
    __shared__ float ml_s[2 * MG_STAGE];
    const int64_t r = blockIdx.x;
    const int64_t t = r / n_heads;
    if (seg_start) {
        const int sg = token_seg[t];
        if (seg_start[sg + 1] - seg_start[sg] != 1) return;
    }
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n = min(n_splits, pos / chunk - lo / chunk + 1);
    const int stride = dv + 2;
    const float* mine = parts + r * n_splits * int64_t(stride);
    const bool staged = n <= MG_STAGE;
    if (staged) {
        for (int i = threadIdx.x; i < 2 * n; i += MG_THREADS) ml_s[i] = mine[(i >> 1) * int64_t(stride) + (i & 1)];
        __syncthreads();
    }
    for (int c = threadIdx.x; c < dv; c += MG_THREADS) {
        float M = -INFINITY, L = 0.0f, O = 0.0f;
#pragma unroll 8
        for (int i = 0; i < n; i++) {
            const float* p = mine + i * int64_t(stride);
            const float v = p[2 + c];
            const float m = staged ? ml_s[2 * i] : p[0], l = staged ? ml_s[2 * i + 1] : p[1];
            float a, b;
            merge_state(M, L, m, l, a, b);
            O = merge_value(O, a, v, b);
        }
        out[r * dv + c] = ib::from_f32<T>(O * (L > 0.0f ? 1.0f / L : 0.0f));
    }
}

constexpr int MG_FLAT_MAX = 512;

// The merge after the tensor-core kernel. One CTA per (token, head), a thread per channel (up to MG_FLAT_MAX). The parts' maxima give one common maximum M; part
// i then weighs exp(m_i - M), computed once per part; the sums of a channel run over the parts in ascending order with
// independent loads, so many are in flight. `ws` holds n_splits weights in shared memory.
template <typename T>
__global__ void __launch_bounds__(MG_FLAT_MAX)
latent_attention_merge_flat_kernel(const float* __restrict__ parts, const int* __restrict__ positions, T* __restrict__ out,
                                   int n_heads, int dv, int window, int n_splits, int chunk, const int* __restrict__ token_seg,
                                   const int* __restrict__ seg_start) {
    ib::pdl_wait();
    extern __shared__ float ws[];                        // [n_splits] weights, then [n_splits] the parts' sums
    __shared__ float red[32];
    const int64_t r = blockIdx.x;
    const int64_t t = r / n_heads;
    if (seg_start) {
        const int sg = token_seg[t];
        if (seg_start[sg + 1] - seg_start[sg] != 1) return;
    }
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n = min(n_splits, pos / chunk - lo / chunk + 1);
    const int stride = dv + 2;
    const float* mine = parts + r * n_splits * int64_t(stride);
    float* ls = ws + n_splits;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float2 ml = *reinterpret_cast<const float2*>(mine + i * int64_t(stride));   // rows start on 8 bytes: dv is even
        ws[i] = ml.x;
        ls[i] = ml.y;
        m = fmaxf(m, ml.x);
    }
    const float M = ib::block_max(m, red);
    for (int i = threadIdx.x; i < n; i += blockDim.x) ws[i] = ws[i] == -INFINITY ? 0.0f : expf(ws[i] - M);
    __syncthreads();
    float L = 0.0f;                                      // every thread adds the same terms in the same order
#pragma unroll 8
    for (int i = 0; i < n; i++) L = fmaf(ls[i], ws[i], L);
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float O = 0.0f;
#pragma unroll 8
        for (int i = 0; i < n; i++) O = fmaf(mine[i * int64_t(stride) + 2 + c], ws[i], O);
        out[r * dv + c] = ib::from_f32<T>(O * inv);
    }
}

// ------------------------------------------------------------------------------------------------
// A head's value up-projection on its latent context, the head's gate and a constant:
//   out[t, h * dv + e] = mult * sigmoid(gates[t, gate_col + h]) * sum_r ctx[t, h, r] * w_uvT[h, r, e]
// (gate_col < 0: no gate). w_uvT is the up-projection transposed per head, so that the columns of a row are
// neighbours (head_product_tile above).
template <typename T>
__global__ void __launch_bounds__(HP_THREADS)
latent_output_kernel(const T* __restrict__ ctx, const T* __restrict__ w_uvT, const float* __restrict__ gates, int64_t gate_ld,
                     int gate_col, float mult, T* __restrict__ out, int64_t n_tokens, int n_heads, int R, int dv, int vec,
                     const int* __restrict__ token_seg, const int* __restrict__ seg_start) {
    ib::pdl_wait();
    constexpr int NT = HP_CL * HpCols<T>::v;
    extern __shared__ __align__(16) float hp_sm[];
    float* a_s = hp_sm;                               // [HP_TOK][R]
    float* red = a_s + HP_TOK * R;                    // [HP_WARPS][HP_TOK][NT]
    const int64_t t0 = int64_t(blockIdx.x) * HP_TOK;
    const int h = blockIdx.y, tid = threadIdx.x;
    const int nt = int(min(int64_t(HP_TOK), n_tokens - t0));
    const unsigned served = tokens_served(t0, nt, token_seg, seg_start);
    if (!served) return;
    for (int i = tid; i < HP_TOK * R; i += HP_THREADS) {
        const int tt = i / R, r = i - tt * R;
        a_s[i] = (served >> tt & 1u) ? ib::to_f32(ctx[((t0 + tt) * n_heads + h) * R + r]) : 0.0f;
    }
    __syncthreads();
    const int n0 = blockIdx.z * NT;
    head_product_tile<T>(a_s, w_uvT + int64_t(h) * R * dv, R, dv, n0, vec != 0, red);
    for (int i = tid; i < HP_TOK * NT; i += HP_THREADS) {
        const int tt = i / NT, n = n0 + (i - tt * NT);
        if (!(served >> tt & 1u) || n >= dv) continue;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < HP_WARPS; w++) s += red[(w * HP_TOK + tt) * NT + (n - n0)];
        const int64_t t = t0 + tt;
        const float gate = gate_col >= 0 ? sigmoid_(gates[t * gate_ld + gate_col + h]) : 1.0f;
        out[(t * n_heads + h) * dv + n] = ib::from_f32<T>(s * gate * mult);
    }
}

// ------------------------------------------------------------------------------------------------
// Router with sigmoid scores. s = sigmoid(logit); the `top` experts with the largest s + correction are chosen (of
// equal ones the lower index); weights[t, e] = mult * s for a chosen expert and 0 for the others. One warp per token.
constexpr int RT_WARPS = 4;

__global__ void __launch_bounds__(RT_WARPS * 32)
route_sigmoid_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int64_t n_tokens, int E, int top,
                     float mult, float* __restrict__ weights, int* __restrict__ chosen) {
    ib::pdl_wait();
    extern __shared__ float rt_sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t t = int64_t(blockIdx.x) * RT_WARPS + warp;
    if (t >= n_tokens) return;
    float* score = rt_sm + warp * 2 * E;              // [E] sigmoid scores
    float* choice = score + E;                        // [E] score + correction; -inf once chosen
    for (int e = lane; e < E; e += 32) {
        const float s = sigmoid_(logits[t * E + e]);
        score[e] = s;
        choice[e] = s + (correction ? correction[e] : 0.0f);
        weights[t * E + e] = 0.0f;
    }
    __syncwarp();
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = E;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi >= E) break;                           // nothing left to choose (NaN or -inf everywhere)
        if (lane == 0) {
            weights[t * E + bi] = score[bi] * mult;
            if (chosen) chosen[t * top + k] = bi;
            choice[bi] = -INFINITY;
        }
        __syncwarp();
    }
}

// Hidden layer of ungated experts: out[t, j] = relu(x[t, j])^2 * scale[t, j / block] (scale absent: 1).
template <typename T>
__global__ void scaled_relu_sq_kernel(const T* __restrict__ x, const float* __restrict__ scale, int64_t n_tokens, int64_t width,
                                      int64_t block, int64_t n_blocks, T* __restrict__ out) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * width) return;
    const int64_t t = i / width, j = i - t * width;
    const float v = fmaxf(ib::to_f32(x[i]), 0.0f);
    const float s = scale ? scale[t * n_blocks + j / block] : 1.0f;
    out[i] = ib::from_f32<T>(v * v * s);
}

// Eight bfloat16 values a thread (width and block multiples of 8). A block whose scale is zero is not read.
__global__ void scaled_relu_sq_vec_kernel(const bf16* __restrict__ x, const float* __restrict__ scale, int64_t n_tokens, int64_t width8,
                                          int64_t block8, int64_t n_blocks, bf16* __restrict__ out) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * width8) return;
    const int64_t t = i / width8, j = i - t * width8;
    const float s = scale ? scale[t * n_blocks + j / block8] : 1.0f;
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (s != 0.0f) {
        const uint4 u = reinterpret_cast<const uint4*>(x)[i];
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&u);
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __bfloat1622float2(hv[k]);
            const float a = fmaxf(f.x, 0.0f), b = fmaxf(f.y, 0.0f);
            ho[k] = __floats2bfloat162_rn(a * a * s, b * b * s);
        }
    }
    reinterpret_cast<uint4*>(out)[i] = r;
}

__global__ void scale_softcap_kernel(float* __restrict__ x, int64_t n, float scale, float cap) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i] * scale;
    x[i] = cap > 0.0f ? cap * tanhf(v / cap) : v;
}

template <typename K>
int allow_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return IB_OK;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
    if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "shared memory of %zu bytes: %s", bytes, cudaGetErrorString(e));
    return IB_OK;
}

}  // namespace

IB_EXPORT int ib_layer_norm(const float* x, const float* w, float eps, int64_t n_rows, int64_t hidden, const int* rows, void* out,
                            int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (hidden <= 0 || hidden > 48 * 1024 / 4) return ib::fail(IB_ERR_ARG, "ib_layer_norm: rows of %lld values are outside 1..12288", (long long)hidden);
    const size_t smem = size_t(hidden) * sizeof(float);
    if (dtype == IB_F32)
        IB_LAUNCH(layer_norm_kernel<float>, unsigned(n_rows), LN_THREADS, smem, x, w, eps, hidden, rows, (float*)out);
    else if (dtype == IB_BF16)
        IB_LAUNCH(layer_norm_kernel<bf16>, unsigned(n_rows), LN_THREADS, smem, x, w, eps, hidden, rows, (bf16*)out);
    else
        return ib::fail(IB_ERR_ARG, "ib_layer_norm: unknown dtype %d", dtype);
    return ib::check_launch("ib_layer_norm");
}

IB_EXPORT int ib_latent_prepare(const float* rows, int64_t ld, int q_col, int q_rank, int kv_col, int kv_rank, int rot_dim,
                                const float* wq, const float* wkv, float eps, const float* cos_t, const float* sin_t, int layout,
                                int n_rot, const int* positions, const int* token_seg, const int* block_table, int64_t max_blocks,
                                void* cq, void* cache, int page_size, int64_t n_pages, int write, int64_t n_tokens, int dtype,
                                int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_rot < 0 || n_rot % 2 || n_rot > rot_dim) return ib::fail(IB_ERR_ARG, "ib_latent_prepare: %d rotated channels of %d", n_rot, rot_dim);
    if (q_rank < 0 || (write && kv_rank <= 0)) return ib::fail(IB_ERR_ARG, "ib_latent_prepare: ranks %d / %d", q_rank, kv_rank);
    if (dtype == IB_F32)
        IB_LAUNCH(latent_prepare_kernel<float>, unsigned(n_tokens), LP_THREADS, 0, rows, ld, q_col, q_rank, kv_col, kv_rank, rot_dim, wq, wkv,
                  eps, cos_t, sin_t, layout, n_rot, positions, token_seg, block_table, max_blocks, (float*)cq, (float*)cache, page_size,
                  n_pages, write, status);
    else if (dtype == IB_BF16)
        IB_LAUNCH(latent_prepare_kernel<bf16>, unsigned(n_tokens), LP_THREADS, 0, rows, ld, q_col, q_rank, kv_col, kv_rank, rot_dim, wq, wkv,
                  eps, cos_t, sin_t, layout, n_rot, positions, token_seg, block_table, max_blocks, (bf16*)cq, (bf16*)cache, page_size,
                  n_pages, write, status);
    else
        return ib::fail(IB_ERR_ARG, "ib_latent_prepare: unknown dtype %d", dtype);
    return ib::check_launch("ib_latent_prepare");
}

namespace {
template <typename T>
size_t head_product_smem(int K) { return (size_t(HP_TOK) * K + size_t(HP_WARPS) * HP_TOK * HP_CL * HpCols<T>::v) * sizeof(float); }
}  // namespace

// `single_start` (the step's seg_start, or null): only tokens that are a segment of their own are served.
IB_EXPORT int ib_latent_query(const void* q, const void* w_uk, const float* cos_t, const float* sin_t, int layout, int n_rot,
                              const int* positions, void* out, int64_t n_tokens, int n_heads, int d, int dr, int R, int dtype,
                              const int* token_seg, const int* single_start, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_heads <= 0 || n_heads > 65535 || d <= 0 || dr < 0 || R <= 0 || n_rot < 0 || n_rot % 2 || n_rot > dr)
        return ib::fail(IB_ERR_ARG, "ib_latent_query: sizes heads %d, %d + %d channels, rank %d, %d rotated", n_heads, d, dr, R, n_rot);
    if (single_start && !token_seg) return ib::fail(IB_ERR_ARG, "ib_latent_query: serving single tokens needs token_seg");
    if (dtype == IB_F32) {
        constexpr int NT = HP_CL * HpCols<float>::v;
        const size_t smem = head_product_smem<float>(d);
        const int rc = allow_smem(latent_query_kernel<float>, smem);
        if (rc) return rc;
        const dim3 grid{blocks_for(n_tokens, HP_TOK), unsigned(n_heads), blocks_for(R, NT)};
        IB_LAUNCH(latent_query_kernel<float>, grid, HP_THREADS, smem, (const float*)q, (const float*)w_uk, cos_t, sin_t, layout, n_rot,
                  positions, (float*)out, n_tokens, n_heads, d, dr, R, int(R % HpCols<float>::v == 0), token_seg, single_start);
    } else if (dtype == IB_BF16) {
        constexpr int NT = HP_CL * HpCols<bf16>::v;
        const size_t smem = head_product_smem<bf16>(d);
        const int rc = allow_smem(latent_query_kernel<bf16>, smem);
        if (rc) return rc;
        const dim3 grid{blocks_for(n_tokens, HP_TOK), unsigned(n_heads), blocks_for(R, NT)};
        IB_LAUNCH(latent_query_kernel<bf16>, grid, HP_THREADS, smem, (const bf16*)q, (const bf16*)w_uk, cos_t, sin_t, layout, n_rot,
                  positions, (bf16*)out, n_tokens, n_heads, d, dr, R, int(R % HpCols<bf16>::v == 0), token_seg, single_start);
    } else
        return ib::fail(IB_ERR_ARG, "ib_latent_query: unknown dtype %d", dtype);
    return ib::check_launch("ib_latent_query");
}

IB_EXPORT int ib_latent_attention_max_dims(int* dk, int* dv) {
    *dk = 1024;
    *dv = 4 * KC;
    return IB_OK;
}

namespace {
template <typename T, int GB, int NC>
int launch_latent_attention(const void* q, const void* cache, const int* block_table, int64_t max_blocks, const int* token_seg,
                            const int* positions, void* out, float* parts, int64_t n_tokens, int n_heads, int group, int dk, int dv,
                            int page_size, int window, float scale, int64_t n_pages, int n_splits, int* status, const int* single_start,
                            cudaStream_t stream) {
    const int dq = (dk + 3) & ~3;
    const size_t smem = size_t(GB * dq + GB * KC + 2 * GMAX) * sizeof(float) + KC * sizeof(int64_t) + size_t(VT) * dv * sizeof(T);
    const int rc = allow_smem(latent_attention_kernel<T, GB, NC>, smem);
    if (rc) return rc;
    const int vec = dk % 8 == 0, vec_v = vec && (dv * sizeof(T)) % 16 == 0;
    const dim3 grid{unsigned(n_tokens), unsigned((n_heads + group - 1) / group), unsigned(n_splits)};
    IB_LAUNCH((latent_attention_kernel<T, GB, NC>), grid, KC, smem, (const T*)q, (const T*)cache, block_table, max_blocks, token_seg,
              positions, (T*)out, parts, n_heads, group, dk, dv, page_size, window, scale, n_pages, n_splits, vec, vec_v, status,
              single_start);
    return IB_OK;
}

template <typename T>
int pick_latent_attention(int gb, int nc, const void* q, const void* cache, const int* block_table, int64_t max_blocks,
                          const int* token_seg, const int* positions, void* out, float* parts, int64_t n_tokens, int n_heads, int group,
                          int dk, int dv, int page_size, int window, float scale, int64_t n_pages, int n_splits, int* status,
                          const int* single_start, cudaStream_t stream) {
#define IB_LA(GB_, NC_)                                                                                                      \
    if (gb == GB_ && nc == NC_)                                                                                              \
        return launch_latent_attention<T, GB_, NC_>(q, cache, block_table, max_blocks, token_seg, positions, out, parts, n_tokens, \
                                                    n_heads, group, dk, dv, page_size, window, scale, n_pages, n_splits, status, single_start, stream);
    IB_LA(1, 1) IB_LA(1, 2) IB_LA(1, 4) IB_LA(2, 1) IB_LA(2, 2) IB_LA(2, 4) IB_LA(4, 1) IB_LA(4, 2) IB_LA(4, 4) IB_LA(8, 1) IB_LA(8, 2) IB_LA(8, 4)
#undef IB_LA
    return ib::fail(IB_ERR_ARG, "ib_latent_attention: no kernel for groups of %d heads and %d channel passes", gb, nc);
}
}  // namespace

// n_splits 1: one CTA per (token, group of heads) walks the token's chunks. n_splits > 1: a token's chunks are spread
// over CTAs; `parts` holds n_tokens * n_heads * n_splits * (dv + 2) floats and the merge kernel follows. n_splits must
// then be at least the number of chunks any token of the step reads.
IB_EXPORT int ib_latent_attention(const void* q, const void* cache, const int* block_table, int64_t max_blocks, const int* token_seg,
                                  const int* positions, void* out, float* parts, int64_t n_tokens, int n_heads, int dk, int dv,
                                  int page_size, int window, float scale, int64_t n_pages, int n_splits, int dtype, int* status,
                                  const int* single_start, int chunk, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (chunk != KC && chunk != TC_KC) return ib::fail(IB_ERR_ARG, "ib_latent_attention: chunks of %d keys", chunk);
    if (n_heads <= 0 || dk <= 0 || dk > 1024 || dv <= 0 || dv > dk || dv > 4 * KC)
        return ib::fail(IB_ERR_ARG, "ib_latent_attention: %d heads, rows of %d with values of %d are outside what the kernel takes", n_heads, dk, dv);
    if (n_splits < 1 || (n_splits > 1 && !parts)) return ib::fail(IB_ERR_ARG, "ib_latent_attention: %d splits need a workspace", n_splits);
    if (n_splits > 65535 || (n_heads + GMAX - 1) / GMAX > 65535) return ib::fail(IB_ERR_ARG, "ib_latent_attention: grid too large");
    if (chunk == TC_KC) {
        // chunks of 64 keys: the tensor-core kernel, which always leaves parts for the merge
        if (dtype != IB_BF16 || dk % 8 || dv % 2 || dv > 512 || !parts)
            return ib::fail(IB_ERR_ARG, "ib_latent_attention: the tensor-core kernel takes bfloat16 rows of a multiple of 8 channels, an even number of values up to 512 and a workspace");
        const int nv = dv <= 64 ? 1 : dv <= 128 ? 2 : dv <= 256 ? 4 : 8;
        const int RS = tc_row_stride(dk);
        const size_t smem = (size_t(TC_HEADS + TC_KC) * RS + 64 * nv + 2 * TC_HEADS * TC_PS) * sizeof(bf16) + 128 * sizeof(float);
        const dim3 grid{unsigned(n_tokens), unsigned((n_heads + TC_HEADS - 1) / TC_HEADS), unsigned(n_splits)};
#define IB_TC(NV_)                                                                                                            \
    if (nv == NV_) {                                                                                                          \
        const int rc = allow_smem(latent_attention_tc_kernel<NV_>, smem);                                                     \
        if (rc) return rc;                                                                                                    \
        IB_LAUNCH(latent_attention_tc_kernel<NV_>, grid, TC_THREADS, smem, (const bf16*)q, (const bf16*)cache, block_table, max_blocks, \
                  token_seg, positions, parts, n_heads, dk, dv, page_size, window, scale, n_pages, n_splits, status, single_start); \
    }
        IB_TC(1) IB_TC(2) IB_TC(4) IB_TC(8)
#undef IB_TC
        const int64_t n_rows = n_tokens * n_heads;
        if (n_rows > 0x7fffffff) return ib::fail(IB_ERR_ARG, "ib_latent_attention: too many rows to merge");
        const size_t merge_smem = size_t(2 * n_splits) * sizeof(float);
        const int rc = allow_smem(latent_attention_merge_flat_kernel<bf16>, merge_smem);
        if (rc) return rc;
        const int merge_threads = dv >= MG_FLAT_MAX ? MG_FLAT_MAX : dv <= MG_THREADS ? MG_THREADS : (dv + 31) / 32 * 32;
        IB_LAUNCH(latent_attention_merge_flat_kernel<bf16>, unsigned(n_rows), merge_threads, merge_smem, parts, positions, (bf16*)out, n_heads,
                  dv, window, n_splits, chunk, token_seg, single_start);
        return ib::check_launch("ib_latent_attention");
    }
    const int group = n_heads < GMAX ? n_heads : GMAX;
    const int gb = group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8;
    const int passes = (dv + KC - 1) / KC, nc = passes <= 1 ? 1 : passes <= 2 ? 2 : 4;
    int rc;
    if (dtype == IB_F32)
        rc = pick_latent_attention<float>(gb, nc, q, cache, block_table, max_blocks, token_seg, positions, out, parts, n_tokens, n_heads,
                                          group, dk, dv, page_size, window, scale, n_pages, n_splits, status, single_start, stream);
    else if (dtype == IB_BF16)
        rc = pick_latent_attention<bf16>(gb, nc, q, cache, block_table, max_blocks, token_seg, positions, out, parts, n_tokens, n_heads,
                                         group, dk, dv, page_size, window, scale, n_pages, n_splits, status, single_start, stream);
    else
        return ib::fail(IB_ERR_ARG, "ib_latent_attention: unknown dtype %d", dtype);
    if (rc) return rc;
    if (n_splits > 1) {
        const int64_t n_rows = n_tokens * n_heads;
        if (n_rows > 0x7fffffff) return ib::fail(IB_ERR_ARG, "ib_latent_attention: too many rows to merge");
        if (dtype == IB_F32)
            IB_LAUNCH(latent_attention_merge_kernel<float>, unsigned(n_rows), MG_THREADS, 0, parts, positions, (float*)out, n_heads, dv,
                      window, n_splits, chunk, token_seg, single_start);
        else
            IB_LAUNCH(latent_attention_merge_kernel<bf16>, unsigned(n_rows), MG_THREADS, 0, parts, positions, (bf16*)out, n_heads, dv,
                      window, n_splits, chunk, token_seg, single_start);
    }
    return ib::check_launch("ib_latent_attention");
}

IB_EXPORT int ib_latent_output(const void* ctx, const void* w_uvT, const float* gates, int64_t gate_ld, int gate_col, float mult,
                               void* out, int64_t n_tokens, int n_heads, int R, int dv, int dtype, const int* token_seg,
                               const int* single_start, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_heads <= 0 || n_heads > 65535 || R <= 0 || dv <= 0) return ib::fail(IB_ERR_ARG, "ib_latent_output: sizes %d heads, rank %d, values %d", n_heads, R, dv);
    if (single_start && !token_seg) return ib::fail(IB_ERR_ARG, "ib_latent_output: serving single tokens needs token_seg");
    if (dtype == IB_F32) {
        constexpr int NT = HP_CL * HpCols<float>::v;
        const size_t smem = head_product_smem<float>(R);
        const int rc = allow_smem(latent_output_kernel<float>, smem);
        if (rc) return rc;
        const dim3 grid{blocks_for(n_tokens, HP_TOK), unsigned(n_heads), blocks_for(dv, NT)};
        IB_LAUNCH(latent_output_kernel<float>, grid, HP_THREADS, smem, (const float*)ctx, (const float*)w_uvT, gates, gate_ld, gate_col, mult,
                  (float*)out, n_tokens, n_heads, R, dv, int(dv % HpCols<float>::v == 0), token_seg, single_start);
    } else if (dtype == IB_BF16) {
        constexpr int NT = HP_CL * HpCols<bf16>::v;
        const size_t smem = head_product_smem<bf16>(R);
        const int rc = allow_smem(latent_output_kernel<bf16>, smem);
        if (rc) return rc;
        const dim3 grid{blocks_for(n_tokens, HP_TOK), unsigned(n_heads), blocks_for(dv, NT)};
        IB_LAUNCH(latent_output_kernel<bf16>, grid, HP_THREADS, smem, (const bf16*)ctx, (const bf16*)w_uvT, gates, gate_ld, gate_col, mult,
                  (bf16*)out, n_tokens, n_heads, R, dv, int(dv % HpCols<bf16>::v == 0), token_seg, single_start);
    } else
        return ib::fail(IB_ERR_ARG, "ib_latent_output: unknown dtype %d", dtype);
    return ib::check_launch("ib_latent_output");
}

IB_EXPORT int ib_route_sigmoid(const float* logits, const float* correction, int64_t n_tokens, int E, int top, float mult,
                               float* weights, int* chosen, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (E <= 0 || top <= 0 || top > E || E > 1024) return ib::fail(IB_ERR_ARG, "ib_route_sigmoid: %d of %d experts", top, E);
    IB_LAUNCH(route_sigmoid_kernel, blocks_for(n_tokens, RT_WARPS), RT_WARPS * 32, size_t(RT_WARPS) * 2 * E * sizeof(float), logits, correction,
              n_tokens, E, top, mult, weights, chosen);
    return ib::check_launch("ib_route_sigmoid");
}

IB_EXPORT int ib_scaled_relu_sq(const void* x, const float* scale, int64_t n_tokens, int64_t width, int64_t block, int64_t n_blocks,
                                void* out, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return IB_OK;
    if (scale && (block <= 0 || n_blocks * block < width)) return ib::fail(IB_ERR_ARG, "ib_scaled_relu_sq: %lld blocks of %lld do not cover %lld columns",
                                                                            (long long)n_blocks, (long long)block, (long long)width);
    if (!scale) { block = width; n_blocks = 1; }
    const int64_t n = n_tokens * width;
    if (dtype == IB_F32)
        IB_LAUNCH(scaled_relu_sq_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)x, scale, n_tokens, width, block, n_blocks, (float*)out);
    else if (dtype == IB_BF16) {
        if (width % 8 == 0 && block % 8 == 0)
            IB_LAUNCH(scaled_relu_sq_vec_kernel, blocks_for(n / 8, 256), 256, 0, (const bf16*)x, scale, n_tokens, width / 8, block / 8, n_blocks, (bf16*)out);
        else
            IB_LAUNCH(scaled_relu_sq_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)x, scale, n_tokens, width, block, n_blocks, (bf16*)out);
    } else
        return ib::fail(IB_ERR_ARG, "ib_scaled_relu_sq: unknown dtype %d", dtype);
    return ib::check_launch("ib_scaled_relu_sq");
}

IB_EXPORT int ib_scale_softcap(float* x, int64_t n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return IB_OK;
    IB_LAUNCH(scale_softcap_kernel, blocks_for(n, 256), 256, 0, x, n, scale, cap);
    return ib::check_launch("ib_scale_softcap");
}
