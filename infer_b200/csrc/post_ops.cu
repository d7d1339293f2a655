// Kernels for layers that normalise AFTER the residual sum, for attention whose queries and keys are normalised per
// head (with a rotation of channel pairs, a temperature on the queries, values that may be the projected keys, and a
// gate per output channel), and for mixers that read mixtures of a token's row with its predecessor's.
//
// Storage of activations is float or bfloat16 (template parameter), arithmetic float. Norms, positions and angles,
// temperatures, decays with their exponentials, and the residual sum are float in both. With float storage these
// kernels are the 32-bit path.
//
// A step's rows are the tokens of several requests ("segments") one after the other: seg_start[s] is the first row
// of segment s, seg_slot[s] the request's state slot. A token's result depends on its own request's earlier tokens
// and state only, and every sum runs in an order fixed by the layer's sizes.
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
__device__ __forceinline__ float silu_(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------------------
// out = y / sqrt(mean(y^2) + eps) * w with y = alpha x + sa a + sb b per row (b may be absent), float; optionally a
// copy of the result in the compute dtype for the next sublayer's first matrix product. One CTA per row; x and out
// may be one buffer (a thread reads and writes the same elements).
template <typename TC>
__global__ void __launch_bounds__(256)
sum_norm_kernel(const float* __restrict__ x, float alpha, const float* __restrict__ a, float sa, const float* __restrict__ b,
                float sb, const float* __restrict__ w, float eps, float* __restrict__ out, TC* __restrict__ copy, int64_t width) {
    ib::pdl_wait();
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const float* xr = x + t * width;
    const float* ar = a + t * width;
    const float* br = b ? b + t * width : nullptr;
    float ss = 0.0f;
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
        float y = fmaf(alpha, xr[i], sa * ar[i]);
        if (br) y = fmaf(sb, br[i], y);
        ss = fmaf(y, y, ss);
    }
    ss = ib::block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / float(width) + eps);
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
        float y = fmaf(alpha, xr[i], sa * ar[i]);
        if (br) y = fmaf(sb, br[i], y);
        const float v = y * f * w[i];
        out[t * width + i] = v;
        if (copy) copy[t * width + i] = ib::from_f32<TC>(v);
    }
}

// ------------------------------------------------------------------------------------------------
// In front of paged attention: projected rows [q (heads x d) | k (kv x d) | v (kv x dv)] from column col0 (the v
// columns absent where the values are the keys as projected) -> q rows for the attention kernel, k and v into the
// token's page. One warp per (token, head of q, k or v). q and k heads are divided by their root mean square over d
// (eps inside the root) and multiplied by a weight [d] that the heads share (wq, wk; null: no norm); then channel
// pairs (2i, 2i + 1) below n_rot turn by the token's position (tables [positions, n_rot / 2]); q is then multiplied
// by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every 0: no temperature). v is stored as projected.
template <typename T>
__global__ void __launch_bounds__(128)
head_prepare_kernel(const T* __restrict__ rows, int64_t ld, int col0, const float* __restrict__ wq, const float* __restrict__ wk,
                    float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_rot, float temp_coef,
                    int temp_every, int values_are_keys, const int* __restrict__ positions, const int* __restrict__ token_seg,
                    const int* __restrict__ block_table, int64_t max_blocks, T* __restrict__ q_out, T* __restrict__ k_cache,
                    T* __restrict__ v_cache, int64_t n_tokens, int n_heads, int n_kv, int d, int dv, int page_size,
                    int write_cache, int64_t n_pages, int* status) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int per_token = n_heads + 2 * n_kv;
    const int64_t wi = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wi >= n_tokens * per_token) return;
    const int64_t t = wi / per_token;
    const int u = int(wi - t * per_token);
    const int pos = positions[t];
    const T* r = rows + t * ld + col0;
    const int nq = n_heads * d, nk = n_kv * d;
    const bool is_q = u < n_heads, is_k = !is_q && u < n_heads + n_kv;
    if (!is_q && !write_cache) return;
    int64_t cache_row = 0;
    if (!is_q) {
        const int page = block_table[int64_t(token_seg[t]) * max_blocks + pos / page_size];
        if (page < 0 || page >= n_pages) {
            if (status && lane == 0) atomicExch(status, 2);
            return;
        }
        const int kvh = is_k ? u - n_heads : u - n_heads - n_kv;
        cache_row = (int64_t(page) * n_kv + kvh) * page_size + pos % page_size;
    }
    if (!is_q && !is_k) {                                  // a value head: as projected
        const int kvh = u - n_heads - n_kv;
        const T* src = values_are_keys ? r + nq + kvh * d : r + nq + nk + kvh * dv;
        T* dst = v_cache + cache_row * dv;
        for (int j = lane; j < dv; j += 32) dst[j] = src[j];
        return;
    }
    const T* src = is_q ? r + u * d : r + nq + (u - n_heads) * d;
    const float* w = is_q ? wq : wk;
    T* dst = is_q ? q_out + t * nq + u * d : k_cache + cache_row * d;
    float f = 1.0f;
    if (w) {
        float ss = 0.0f;
        for (int j = lane; j < d; j += 32) { const float v = ib::to_f32(src[j]); ss = fmaf(v, v, ss); }
        ss = ib::warp_sum(ss);
        f = 1.0f / sqrtf(ss / float(d) + eps);
    }
    float mult = 1.0f;
    if (is_q && temp_every > 0) mult = 1.0f + temp_coef * logf(float((pos + 1) / temp_every + 1));
    const int half = n_rot / 2;
    for (int p = lane; 2 * p < d; p += 32) {
        const int j = 2 * p;
        float a = ib::to_f32(src[j]) * f, b = j + 1 < d ? ib::to_f32(src[j + 1]) * f : 0.0f;
        if (w) { a *= w[j]; if (j + 1 < d) b *= w[j + 1]; }
        if (p < half) {
            const float c = cos_t[int64_t(pos) * half + p], s = sin_t[int64_t(pos) * half + p];
            const float a2 = a * c - b * s, b2 = b * c + a * s;
            a = a2; b = b2;
        }
        dst[j] = ib::from_f32<T>(a * mult);
        if (j + 1 < d) dst[j + 1] = ib::from_f32<T>(b * mult);
    }
}

// ctx[t, i] *= sigmoid(rows[t, gate_col + i]) for i < width, in place.
template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ ctx, const T* __restrict__ rows, int64_t ld, int64_t gate_col, int64_t width, int64_t n) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / width, c = i - t * width;
    ctx[i] = ib::from_f32<T>(ib::to_f32(ctx[i]) * sigmoid_(ib::to_f32(rows[t * ld + gate_col + c])));
}

// silu of columns [col0, col0 + width) of float rows, in place.
__global__ void silu_rows_kernel(float* __restrict__ rows, int64_t ld, int64_t col0, int64_t width, int64_t n) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / width, c = i - t * width;
    float* p = rows + t * ld + col0 + c;
    *p = silu_(*p);
}

// ------------------------------------------------------------------------------------------------
// Mixtures of a token's row with its predecessor's: out[m][t][c] = x[t][c] + (x'[t][c] - x[t][c]) * mu[m][c], where
// x' is the row of the token before (the request's kept row `last` [slots, width] for a segment's first token: zeros
// for a new request). With write_state the thread that read a segment's kept row replaces it by the segment's last row.
template <typename TC>
__global__ void shift_mix_kernel(const float* __restrict__ x, float* __restrict__ last, const float* __restrict__ mu, int n_mix,
                                 const int* __restrict__ token_seg, const int* __restrict__ seg_start,
                                 const int* __restrict__ seg_slot, TC* __restrict__ out, int64_t n_tokens, int64_t width,
                                 int write_state) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * width) return;
    const int64_t t = i / width, c = i - t * width;
    const int s = token_seg[t];
    const float h = x[i];
    float before;
    if (t == seg_start[s]) {
        float* kept = last + int64_t(seg_slot[s]) * width + c;
        before = *kept;
        if (write_state) *kept = x[(int64_t(seg_start[s + 1]) - 1) * width + c];
    } else {
        before = x[i - width];
    }
    const float diff = before - h;
    for (int m = 0; m < n_mix; m++) out[(int64_t(m) * n_tokens + t) * width + c] = ib::from_f32<TC>(fmaf(diff, mu[m * width + c], h));
}

// decay[t, c] = exp(-exp(bias[c] + sum_r up[r, c] * tanh(low[t, r]))), float: a decay per channel and token through a
// low rank. low: columns [low_col, low_col + rank) of the rows (float or bfloat16); up stored [rank, channels].
template <typename T>
__global__ void __launch_bounds__(256)
double_exp_decay_kernel(const T* __restrict__ rows, int64_t ld, int low_col, int rank, const float* __restrict__ up,
                        const float* __restrict__ bias, float* __restrict__ decay, int channels) {
    ib::pdl_wait();
    extern __shared__ float low[];
    const int64_t t = blockIdx.y;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) low[r] = tanhf(ib::to_f32(rows[t * ld + low_col + r]));
    __syncthreads();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float z = bias ? bias[c] : 0.0f;
    for (int r = 0; r < rank; r++) z = fmaf(up[int64_t(r) * channels + c], low[r], z);
    decay[t * channels + c] = expf(-expf(z));
}

// One warp per (token, group of `size` channels): out = o / sqrt(mean(o^2) + eps) * w [* act(gate)], o float
// [tokens, groups * size]; w [groups * size] (null: no weight); the gate's logits are columns gate_col + g size + j
// of rows `gate` (leading dimension ldg); act: 1 silu, 2 sigmoid, 0 the logits are multipliers as they are.
template <typename TG, typename TOut>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                       const TG* __restrict__ gate, int64_t ldg, int64_t gate_col, int act, TOut* __restrict__ out,
                                       int64_t n_rows, int n_groups, int size) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t r = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int64_t t = r / n_groups;
    const int g = int(r - t * n_groups);
    const float* x = o + r * size;
    float ss = 0.0f;
    for (int j = lane; j < size; j += 32) ss = fmaf(x[j], x[j], ss);
    ss = ib::warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / float(size) + eps);
    for (int j = lane; j < size; j += 32) {
        float y = x[j] * f;
        if (w) y *= w[int64_t(g) * size + j];
        if (gate) {
            const float z = ib::to_f32(gate[t * ldg + gate_col + int64_t(g) * size + j]);
            y *= act == 1 ? silu_(z) : (act == 2 ? sigmoid_(z) : z);
        }
        out[r * size + j] = ib::from_f32<TOut>(y);
    }
}

// relu(x)^2 of columns [col0, col0 + width) of the rows -> contiguous [tokens, width].
template <typename T>
__global__ void relu_sq_kernel(const T* __restrict__ rows, int64_t ld, int64_t col0, int64_t width, T* __restrict__ out, int64_t n) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / width, c = i - t * width;
    const float v = fmaxf(ib::to_f32(rows[t * ld + col0 + c]), 0.0f);
    out[i] = ib::from_f32<T>(v * v);
}

// The same for bfloat16 rows whose sizes and addresses allow 16-byte accesses: eight columns a thread.
__global__ void relu_sq_vec_kernel(const bf16* __restrict__ rows, int64_t ld, int64_t col0, int64_t width8, bf16* __restrict__ out, int64_t n8) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const int64_t t = i / width8, c = (i - t * width8) * 8;
    const uint4 in = *reinterpret_cast<const uint4*>(rows + t * ld + col0 + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
    uint4 res;
    __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 f = __bfloat1622float2(h[k]);
        const float a = fmaxf(f.x, 0.0f), b = fmaxf(f.y, 0.0f);
        rh[k] = __floats2bfloat162_rn(a * a, b * b);
    }
    *reinterpret_cast<uint4*>(out + i * 8) = res;
}

// group_norm_gate with one CTA per (token, group), for groups of many channels (all heads of a token at once): the
// same result as the warp form up to the order of the sum of squares; which form runs depends on the group's size only.
template <typename TG, typename TOut>
__global__ void __launch_bounds__(256)
group_norm_gate_wide_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const TG* __restrict__ gate,
                            int64_t ldg, int64_t gate_col, int act, TOut* __restrict__ out, int n_groups, int size) {
    ib::pdl_wait();
    __shared__ float red[32];
    const int64_t r = blockIdx.x;
    const int64_t t = r / n_groups;
    const int g = int(r - t * n_groups);
    const float* x = o + r * size;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < size; j += blockDim.x) ss = fmaf(x[j], x[j], ss);
    ss = ib::block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / float(size) + eps);
    for (int j = threadIdx.x; j < size; j += blockDim.x) {
        float y = x[j] * f;
        if (w) y *= w[int64_t(g) * size + j];
        if (gate) {
            const float z = ib::to_f32(gate[t * ldg + gate_col + int64_t(g) * size + j]);
            y *= act == 1 ? silu_(z) : (act == 2 ? sigmoid_(z) : z);
        }
        out[r * size + j] = ib::from_f32<TOut>(y);
    }
}

// double_exp_decay for TT tokens a CTA: a thread keeps one channel's column of `up` in flight once for all of them.
constexpr int DECAY_TOKENS = 8;
template <typename T>
__global__ void __launch_bounds__(256)
double_exp_decay_tokens_kernel(const T* __restrict__ rows, int64_t ld, int low_col, int rank, const float* __restrict__ up,
                               const float* __restrict__ bias, float* __restrict__ decay, int channels, int64_t n_tokens) {
    ib::pdl_wait();
    extern __shared__ float low[];                          // [DECAY_TOKENS][rank]
    const int64_t t0 = int64_t(blockIdx.y) * DECAY_TOKENS;
    const int nt = int(min(int64_t(DECAY_TOKENS), n_tokens - t0));
    for (int i = threadIdx.x; i < nt * rank; i += blockDim.x) {
        const int tt = i / rank, r = i - tt * rank;
        low[i] = tanhf(ib::to_f32(rows[(t0 + tt) * ld + low_col + r]));
    }
    __syncthreads();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float z[DECAY_TOKENS];
    const float b = bias ? bias[c] : 0.0f;
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; tt++) z[tt] = b;
    for (int r = 0; r < rank; r++) {
        const float u = up[int64_t(r) * channels + c];
#pragma unroll
        for (int tt = 0; tt < DECAY_TOKENS; tt++)
            if (tt < nt) z[tt] = fmaf(u, low[tt * rank + r], z[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; tt++)
        if (tt < nt) decay[(t0 + tt) * channels + c] = expf(-expf(z[tt]));
}

}  // namespace

// ================================================================================================
// C entry points. dtype arguments: 0 = float, 1 = bfloat16.

IB_EXPORT int ib_sum_norm(const float* x, float alpha, const float* a, float sa, const float* b, float sb, const float* w, float eps,
                          float* out, void* copy, int copy_dtype, int64_t n_tokens, int64_t width, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return IB_OK;
    if (!x || !a || !w || !out) return ib::fail(IB_ERR_ARG, "ib_sum_norm: rows, a term, the weight and the result are needed");
    if (copy && copy_dtype == IB_BF16)
        IB_LAUNCH(sum_norm_kernel<bf16>, unsigned(n_tokens), 256, 0, x, alpha, a, sa, b, sb, w, eps, out, (bf16*)copy, width);
    else if (!copy || copy_dtype == IB_F32)
        IB_LAUNCH(sum_norm_kernel<float>, unsigned(n_tokens), 256, 0, x, alpha, a, sa, b, sb, w, eps, out, (float*)copy, width);
    else
        return ib::fail(IB_ERR_ARG, "ib_sum_norm: unknown dtype %d", copy_dtype);
    return ib::check_launch("ib_sum_norm");
}

IB_EXPORT int ib_head_prepare(const void* rows, int64_t ld, int col0, const float* wq, const float* wk, float eps, const float* cos_t,
                              const float* sin_t, int n_rot, float temp_coef, int temp_every, int values_are_keys,
                              const int* positions, const int* token_seg, const int* block_table, int64_t max_blocks, void* q_out,
                              void* k_cache, void* v_cache, int64_t n_tokens, int n_heads, int n_kv, int d, int dv, int page_size,
                              int write_cache, int64_t n_pages, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv <= 0 || d <= 0 || dv <= 0 || page_size <= 0)
        return ib::fail(IB_ERR_ARG, "ib_head_prepare: bad sizes");
    if (n_rot < 0 || n_rot % 2 || n_rot > d || (n_rot > 0 && (!cos_t || !sin_t)))
        return ib::fail(IB_ERR_ARG, "ib_head_prepare: %d rotated channels of %d need tables and an even count", n_rot, d);
    if (values_are_keys && dv != d) return ib::fail(IB_ERR_ARG, "ib_head_prepare: values that are the keys have the keys' size");
    const int64_t warps = n_tokens * (n_heads + 2 * n_kv);
#define IB_HP(TT)                                                                                                                 \
    IB_LAUNCH(head_prepare_kernel<TT>, blocks_for(warps, 4), 128, 0, (const TT*)rows, ld, col0, wq, wk, eps, cos_t, sin_t, n_rot,  \
              temp_coef, temp_every, values_are_keys, positions, token_seg, block_table, max_blocks, (TT*)q_out, (TT*)k_cache,    \
              (TT*)v_cache, n_tokens, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status)
    if (dtype == IB_F32) IB_HP(float);
    else if (dtype == IB_BF16) IB_HP(bf16);
    else return ib::fail(IB_ERR_ARG, "ib_head_prepare: unknown dtype %d", dtype);
#undef IB_HP
    return ib::check_launch("ib_head_prepare");
}

IB_EXPORT int ib_gate_mul(void* ctx, const void* rows, int64_t ld, int64_t gate_col, int64_t width, int64_t n_tokens, int dtype,
                          cudaStream_t stream) {
    const int64_t n = n_tokens * width;
    if (n <= 0) return IB_OK;
    if (dtype == IB_F32) IB_LAUNCH(gate_mul_kernel<float>, blocks_for(n, 256), 256, 0, (float*)ctx, (const float*)rows, ld, gate_col, width, n);
    else if (dtype == IB_BF16) IB_LAUNCH(gate_mul_kernel<bf16>, blocks_for(n, 256), 256, 0, (bf16*)ctx, (const bf16*)rows, ld, gate_col, width, n);
    else return ib::fail(IB_ERR_ARG, "ib_gate_mul: unknown dtype %d", dtype);
    return ib::check_launch("ib_gate_mul");
}

IB_EXPORT int ib_silu_rows(float* rows, int64_t ld, int64_t col0, int64_t width, int64_t n_tokens, cudaStream_t stream) {
    const int64_t n = n_tokens * width;
    if (n <= 0) return IB_OK;
    IB_LAUNCH(silu_rows_kernel, blocks_for(n, 256), 256, 0, rows, ld, col0, width, n);
    return ib::check_launch("ib_silu_rows");
}

IB_EXPORT int ib_shift_mix(const float* x, float* last, const float* mu, int n_mix, const int* token_seg, const int* seg_start,
                           const int* seg_slot, void* out, int out_dtype, int64_t n_tokens, int64_t width, int write_state,
                           cudaStream_t stream) {
    const int64_t n = n_tokens * width;
    if (n <= 0 || n_mix <= 0) return IB_OK;
    if (out_dtype == IB_F32)
        IB_LAUNCH(shift_mix_kernel<float>, blocks_for(n, 256), 256, 0, x, last, mu, n_mix, token_seg, seg_start, seg_slot, (float*)out, n_tokens, width, write_state);
    else if (out_dtype == IB_BF16)
        IB_LAUNCH(shift_mix_kernel<bf16>, blocks_for(n, 256), 256, 0, x, last, mu, n_mix, token_seg, seg_start, seg_slot, (bf16*)out, n_tokens, width, write_state);
    else
        return ib::fail(IB_ERR_ARG, "ib_shift_mix: unknown dtype %d", out_dtype);
    return ib::check_launch("ib_shift_mix");
}

IB_EXPORT int ib_double_exp_decay(const void* rows, int64_t ld, int low_col, int rank, const float* up, const float* bias, float* decay,
                                  int64_t n_tokens, int channels, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return IB_OK;
    if (rank <= 0 || rank > 8192 || n_tokens > 2147483647) return ib::fail(IB_ERR_ARG, "ib_double_exp_decay: a rank of %d", rank);
    // A few tokens (a decode step): a CTA per (token, 256 channels), so that there are CTAs enough.
    if (n_tokens < 8 * DECAY_TOKENS) {
        const dim3 grid1{blocks_for(channels, 256), unsigned(n_tokens), 1u};
        if (dtype == IB_F32)
            IB_LAUNCH(double_exp_decay_kernel<float>, grid1, 256, rank * sizeof(float), (const float*)rows, ld, low_col, rank, up, bias, decay, channels);
        else if (dtype == IB_BF16)
            IB_LAUNCH(double_exp_decay_kernel<bf16>, grid1, 256, rank * sizeof(float), (const bf16*)rows, ld, low_col, rank, up, bias, decay, channels);
        else
            return ib::fail(IB_ERR_ARG, "ib_double_exp_decay: unknown dtype %d", dtype);
        return ib::check_launch("ib_double_exp_decay");
    }
    // Otherwise groups of DECAY_TOKENS tokens on the grid's y axis. Each channel's sum runs over the rank in ascending
    // order whatever the grouping: a token's bits do not depend on its neighbours or on which form ran.
    const int64_t groups = (n_tokens + DECAY_TOKENS - 1) / DECAY_TOKENS;
    if (groups > 65535 || size_t(DECAY_TOKENS) * rank * sizeof(float) > 48 * 1024)
        return ib::fail(IB_ERR_ARG, "ib_double_exp_decay: %lld tokens at rank %d", (long long)n_tokens, rank);
    const dim3 grid{blocks_for(channels, 256), unsigned(groups), 1u};
    const size_t smem = size_t(DECAY_TOKENS) * rank * sizeof(float);
    if (dtype == IB_F32)
        IB_LAUNCH(double_exp_decay_tokens_kernel<float>, grid, 256, smem, (const float*)rows, ld, low_col, rank, up, bias, decay, channels, n_tokens);
    else if (dtype == IB_BF16)
        IB_LAUNCH(double_exp_decay_tokens_kernel<bf16>, grid, 256, smem, (const bf16*)rows, ld, low_col, rank, up, bias, decay, channels, n_tokens);
    else
        return ib::fail(IB_ERR_ARG, "ib_double_exp_decay: unknown dtype %d", dtype);
    return ib::check_launch("ib_double_exp_decay");
}

IB_EXPORT int ib_group_norm_gate(const float* o, const float* w, float eps, const void* gate, int64_t ldg, int64_t gate_col,
                                 int gate_dtype, int act, void* out, int out_dtype, int64_t n_tokens, int n_groups, int size,
                                 cudaStream_t stream) {
    const int64_t rows = n_tokens * n_groups;
    if (rows <= 0 || size <= 0) return IB_OK;
    const bool wide = size >= 512;                          // (by the group's size only, never by the number of rows)
    const unsigned grid = wide ? unsigned(rows) : blocks_for(rows, 8);
#define IB_GN(TG, TO)                                                                                                               \
    do {                                                                                                                            \
        if (wide) IB_LAUNCH((group_norm_gate_wide_kernel<TG, TO>), grid, 256, 0, o, w, eps, (const TG*)gate, ldg, gate_col, act, (TO*)out, n_groups, size); \
        else IB_LAUNCH((group_norm_gate_kernel<TG, TO>), grid, 256, 0, o, w, eps, (const TG*)gate, ldg, gate_col, act, (TO*)out, rows, n_groups, size);     \
    } while (0)
    if (!gate || gate_dtype == IB_F32) {
        if (out_dtype == IB_F32) IB_GN(float, float);
        else if (out_dtype == IB_BF16) IB_GN(float, bf16);
        else return ib::fail(IB_ERR_ARG, "ib_group_norm_gate: unknown dtype %d", out_dtype);
    } else if (gate_dtype == IB_BF16) {
        if (out_dtype == IB_F32) IB_GN(bf16, float);
        else if (out_dtype == IB_BF16) IB_GN(bf16, bf16);
        else return ib::fail(IB_ERR_ARG, "ib_group_norm_gate: unknown dtype %d", out_dtype);
    } else {
        return ib::fail(IB_ERR_ARG, "ib_group_norm_gate: unknown gate dtype %d", gate_dtype);
    }
#undef IB_GN
    return ib::check_launch("ib_group_norm_gate");
}

IB_EXPORT int ib_relu_sq(const void* rows, int64_t ld, int64_t col0, int64_t width, void* out, int64_t n_tokens, int dtype,
                         cudaStream_t stream) {
    const int64_t n = n_tokens * width;
    if (n <= 0) return IB_OK;
    if (dtype == IB_F32) IB_LAUNCH(relu_sq_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)rows, ld, col0, width, (float*)out, n);
    else if (dtype == IB_BF16 && width % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 && !((uintptr_t(rows) | uintptr_t(out)) & 15))
        // (chosen by sizes and addresses, never by the number of rows)
        IB_LAUNCH(relu_sq_vec_kernel, blocks_for(n / 8, 256), 256, 0, (const bf16*)rows, ld, col0, width / 8, (bf16*)out, n / 8);
    else if (dtype == IB_BF16) IB_LAUNCH(relu_sq_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)rows, ld, col0, width, (bf16*)out, n);
    else return ib::fail(IB_ERR_ARG, "ib_relu_sq: unknown dtype %d", dtype);
    return ib::check_launch("ib_relu_sq");
}
