// Kernels for layers that normalise what a sublayer returns, for linear recurrences with a matrix state per head
// (a decay per key channel; the gated delta rule), for whole-row query/key norms in front of paged attention, and
// for routed feed-forwards (router, clipped gated activations).
//
// Storage of activations is float or bfloat16 (template parameter), arithmetic float. Norms, routers, decays and
// their logarithms, step sizes, unit norms, recurrent state and the residual sum are float in both. With float
// storage these kernels are the 32-bit path.
//
// A step's rows are the tokens of several requests ("segments") one after the other: seg_start[s] is the first row
// of segment s, seg_slot[s] the request's state slot. A token's result depends on its own request's earlier tokens
// and state only, and every sum runs in an order fixed by the layer's sizes: results do not depend on how a prompt
// was cut or on what else is in the step.
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
__device__ __forceinline__ float softplus_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float log_sigmoid_(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------------------------------------
// out = x + y / sqrt(mean(y^2) + eps) * w per row (x absent: the norm alone), float; optionally a copy of the result
// in the compute dtype for the next sublayer's first matrix product. One CTA per row. x and out may be one buffer.
template <typename TC>
__global__ void __launch_bounds__(256)
norm_add_kernel(const float* x, const float* __restrict__ y, const float* __restrict__ w, float eps, float* out,
                TC* __restrict__ copy, int64_t width) {
    ib::pdl_wait();
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const float* yr = y + t * width;
    float ss = 0.0f;
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
    ss = ib::block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / float(width) + eps);
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
        float v = yr[i] * f * w[i];
        if (x) v += x[t * width + i];
        out[t * width + i] = v;
        if (copy) copy[t * width + i] = ib::from_f32<TC>(v);
    }
}

// Float rows in the compute dtype (for a sublayer that reads the residual stream itself).
template <typename TC>
__global__ void cast_rows_kernel(const float* __restrict__ x, TC* __restrict__ out, int64_t n) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = ib::from_f32<TC>(x[i]);
}

// m = sa * a / rms(a) * wa + sb * b / rms(b) * wb per row (two sublayers side by side, each normalised over the
// width); then, with wo given, out = x + m / rms(m) * wo and the compute-dtype copy, as norm_add does: the layer's
// whole tail in one pass over the rows. Without wo: out = m.
template <typename TC>
__global__ void __launch_bounds__(256)
dual_norm_sum_kernel(const float* __restrict__ a, const float* __restrict__ wa, float sa, const float* __restrict__ b,
                     const float* __restrict__ wb, float sb, float eps, const float* x, const float* __restrict__ wo,
                     float eps_o, float* out, TC* __restrict__ copy, int64_t width) {
    ib::pdl_wait();
    extern __shared__ float row[];           // [width]
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const float* ar = a + t * width;
    const float* br = b + t * width;
    float s1 = 0.0f, s2 = 0.0f;
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
        s1 = fmaf(ar[i], ar[i], s1);
        s2 = fmaf(br[i], br[i], s2);
    }
    s1 = ib::block_sum(s1, red);
    s2 = ib::block_sum(s2, red);
    const float fa = sa / sqrtf(s1 / float(width) + eps), fb = sb / sqrtf(s2 / float(width) + eps);
    float s3 = 0.0f;
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
        const float m = ar[i] * fa * wa[i] + br[i] * fb * wb[i];
        row[i] = m;
        s3 = fmaf(m, m, s3);
    }
    if (!wo) {
        for (int64_t i = threadIdx.x; i < width; i += blockDim.x) out[t * width + i] = row[i];
        return;
    }
    s3 = ib::block_sum(s3, red);
    const float fo = 1.0f / sqrtf(s3 / float(width) + eps_o);
    for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
        float v = row[i] * fo * wo[i];
        if (x) v += x[t * width + i];
        out[t * width + i] = v;
        if (copy) copy[t * width + i] = ib::from_f32<TC>(v);
    }
}

// ------------------------------------------------------------------------------------------------
// Gated activations of a feed-forward's hidden layer: columns [gate_col, gate_col + width) and [up_col, ...) of the
// rows -> out [tokens, width] contiguous.
//   kind 0: gelu_tanh(g) * u
//   kind 1: g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(slope * g') * (u' + 1)
//   kind 2: g * sigmoid(g) * u
// Columns are cut into blocks of `group` (an expert's hidden size): block e of token t is multiplied by
// scale[t * n_groups + e] (a router's weight, zero for an expert the token does not use); columns from
// n_groups * group on (a shared expert) are not scaled and use limit2.
template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ rows, int64_t ld, int64_t gate_col, int64_t up_col, int64_t width,
                               int kind, float limit, float limit2, float slope, const float* __restrict__ scale,
                               int64_t group, int64_t n_groups, T* __restrict__ out, int64_t n) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / width, c = i - t * width;
    float g = ib::to_f32(rows[t * ld + gate_col + c]);
    float u = ib::to_f32(rows[t * ld + up_col + c]);
    float y;
    if (kind == 0) {
        y = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    } else if (kind == 2) {
        const int64_t e = group > 0 ? c / group : 0;
        y = silu_(g) * u;
        if (scale && e < n_groups) y *= scale[t * n_groups + e];
    } else {
        const int64_t e = group > 0 ? c / group : 0;
        const float lim = (group > 0 && e >= n_groups) ? limit2 : limit;
        g = fminf(g, lim);
        u = fminf(fmaxf(u, -lim), lim);
        y = g * sigmoid_(slope * g) * (u + 1.0f);
        if (scale && e < n_groups) y *= scale[t * n_groups + e];
    }
    out[i] = ib::from_f32<T>(y);
}

// The same for bfloat16 rows whose sizes and addresses allow 16-byte accesses: eight columns a thread (they lie in one
// block, since `group` is a multiple of eight).
__global__ void glu_act_vec_kernel(const bf16* __restrict__ rows, int64_t ld, int64_t gate_col, int64_t up_col, int64_t width8,
                                   int kind, float limit, float limit2, float slope, const float* __restrict__ scale,
                                   int64_t group, int64_t n_groups, bf16* __restrict__ out, int64_t n8) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const int64_t t = i / width8, c = (i - t * width8) * 8;
    const uint4 gu = *reinterpret_cast<const uint4*>(rows + t * ld + gate_col + c);
    const uint4 uu = *reinterpret_cast<const uint4*>(rows + t * ld + up_col + c);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uu);
    const int64_t e = group > 0 ? c / group : 0;
    const float lim = (group > 0 && e >= n_groups) ? limit2 : limit;
    const float sc = (kind != 0 && scale && e < n_groups) ? scale[t * n_groups + e] : 1.0f;
    uint4 res;
    __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 g2 = __bfloat1622float2(gh[k]), u2 = __bfloat1622float2(uh[k]);
        float y[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            float g = j ? g2.y : g2.x, u = j ? u2.y : u2.x;
            if (kind == 0) {
                y[j] = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
            } else if (kind == 2) {
                y[j] = silu_(g) * u * sc;
            } else {
                g = fminf(g, lim);
                u = fminf(fmaxf(u, -lim), lim);
                y[j] = g * sigmoid_(slope * g) * (u + 1.0f);
                if (scale && e < n_groups) y[j] *= sc;
            }
        }
        rh[k] = __floats2bfloat162_rn(y[0], y[1]);
    }
    *reinterpret_cast<uint4*>(out + i * 8) = res;
}

// ------------------------------------------------------------------------------------------------
// Router: scores = softmax(logits) over all experts; experts form n_groups groups of neighbours, a group's score is
// its largest; only experts of the `keep` best groups can be chosen; the `top` largest of those are chosen (ties:
// the lower index); their weights are their scores divided by (their sum + sum_eps). One warp per token.
// weights [tokens, experts]: a chosen expert's weight, zero elsewhere. chosen [tokens, top] (optional): the indices.
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, int64_t n_tokens, int n_experts, int top, int n_groups, int keep,
             float sum_eps, float* __restrict__ weights, int* __restrict__ chosen) {
    ib::pdl_wait();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t t = int64_t(blockIdx.x) * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* s = sm + warp * (n_experts + n_groups);          // scores; a chosen expert's score becomes -(1 + score)
    float* gs = s + n_experts;                               // group scores; -1: a kept group, -2: not kept
    const float* z = logits + t * n_experts;
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, z[e]);
    mx = ib::warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < n_experts; e += 32) {
        const float v = expf(z[e] - mx);
        s[e] = v;
        sum += v;
    }
    sum = ib::warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < n_experts; e += 32) s[e] = s[e] / sum;
    __syncwarp();
    const int per = n_experts / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
        float m = -1.0f;
        for (int j = 0; j < per; j++) m = fmaxf(m, s[g * per + j]);
        gs[g] = m;
    }
    __syncwarp();
    for (int r = 0; r < keep; r++) {
        float best = -1.0f;
        int at = 0x7fffffff;
        for (int g = lane; g < n_groups; g += 32)
            if (gs[g] > best) { best = gs[g]; at = g; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0 && at < n_groups) gs[at] = -1.0f - 1.0f;   // kept (marked below as -1 after the loop)
        __syncwarp();
    }
    // a kept group now holds -2, every other its score >= 0
    float total = 0.0f;
    for (int r = 0; r < top; r++) {
        float best = -1.0f;
        int at = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32)
            if (gs[e / per] < -1.5f && s[e] > best) { best = s[e]; at = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at < n_experts) {
            total += best;
            if (lane == 0) {
                s[at] = -1.0f - best;
                if (chosen) chosen[t * top + r] = at;
            }
        } else if (lane == 0 && chosen) {
            chosen[t * top + r] = -1;
        }
        __syncwarp();
    }
    const float inv = 1.0f / (total + sum_eps);
    for (int e = lane; e < n_experts; e += 32) weights[t * n_experts + e] = s[e] < 0.0f ? (-1.0f - s[e]) * inv : 0.0f;
}

// ------------------------------------------------------------------------------------------------
// In front of paged attention: projected rows [q | k | v] (q at column col0) -> q rows for the attention kernel, k and
// v into the token's page. q is normalised over ALL its heads * d channels at once, with a weight per channel (wq),
// k likewise (wk); a null weight leaves that projection as it is. One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256)
rownorm_store_kernel(const T* __restrict__ rows, int64_t ld, int col0, const float* __restrict__ wq,
                     const float* __restrict__ wk, float eps, const int* __restrict__ positions,
                     const int* __restrict__ token_seg, const int* __restrict__ block_table, int64_t max_blocks,
                     T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, int n_heads, int n_kv, int d,
                     int dv, int page_size, int write_cache, int64_t n_pages, int* status) {
    ib::pdl_wait();
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const int nq = n_heads * d, nk = n_kv * d, nv = n_kv * dv;
    const T* r = rows + t * ld + col0;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = ib::to_f32(r[i]); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = ib::to_f32(r[nq + i]); sk = fmaf(v, v, sk); }
    sq = ib::block_sum(sq, red);
    sk = ib::block_sum(sk, red);
    const float fq = 1.0f / sqrtf(sq / float(nq) + eps), fk = 1.0f / sqrtf(sk / float(nk) + eps);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const float v = ib::to_f32(r[i]);
        q_out[t * nq + i] = wq ? ib::from_f32<T>(v * fq * wq[i]) : r[i];
    }
    if (!write_cache) return;
    const int pos = positions[t];
    const int page = block_table[int64_t(token_seg[t]) * max_blocks + pos / page_size];
    if (page < 0 || page >= n_pages) {
        if (status && threadIdx.x == 0) atomicExch(status, 2);
        return;
    }
    const int place = pos % page_size;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int h = i / d, j = i - h * d;
        const float v = ib::to_f32(r[nq + i]);
        k_cache[((int64_t(page) * n_kv + h) * page_size + place) * d + j] = wk ? ib::from_f32<T>(v * fk * wk[i]) : r[nq + i];
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int h = i / dv, j = i - h * dv;
        v_cache[((int64_t(page) * n_kv + h) * page_size + place) * dv + j] = r[nq + nk + i];
    }
}

// ------------------------------------------------------------------------------------------------
// Paged attention of single tokens with a window, a bias per (distance, head) and a sink, keys split over CTAs: a
// decoded token of a windowed layer reads a few hundred keys, which one CTA per (token, head) walks too slowly.
// One CTA per (token, kv head, chunk of KC keys aligned to absolute multiples of KC); its `group` query heads share
// every key and value row that is read. Score phase: a thread per key (16-byte loads of its row where the sizes
// allow), the group's queries in shared memory; softmax per head by a warp; value phase: a thread per channel.
// A chunk leaves (maximum, sum, unnormalised context) per head in the workspace; the merge kernel adds a token's
// chunks in ascending order, counts the sink once and divides. What a token's result depends on is (window, position)
// only. `single_only` (a step's seg_start): tokens of longer segments are skipped (another kernel's).
// With keep_first > 0 a windowed query also sees the keys below keep_first: their chunks come first in a token's list of
// chunks, then the window's. With `slopes` [heads], slopes[h] * (position - key) is taken off the scaled score.
constexpr int KC = 128;
constexpr int GMAX = 16;
constexpr int VT = 32;                 // value rows staged at a time

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

// GB: the group's size rounded up to 1, 2, 4, 8 or 16 (the loops over a group's heads are unrolled to it).
template <typename T, int GB>
__global__ void __launch_bounds__(KC)
split_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int* __restrict__ block_table, int64_t max_blocks, const int* __restrict__ token_seg,
                       const int* __restrict__ positions, const int* __restrict__ single_only, float* __restrict__ parts,
                       int n_heads, int n_kv, int d, int dv, int page_size, int window, float scale, int64_t n_pages,
                       const float* __restrict__ dist_bias, int bias_len, int n_chunks, int vec, int vec_v, int* status,
                       int keep_first, const float* __restrict__ slopes) {
    ib::pdl_wait();
    const int64_t t = blockIdx.x;
    const int g = blockIdx.y, ci = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sg = token_seg[t];
    if (single_only && single_only[sg + 1] - single_only[sg] > 1) return;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int keep_end = min(keep_first, lo);                    // keys below it are seen although the window has passed
    const int nk = min((keep_end + KC - 1) / KC, lo / KC);      // chunks of kept keys that lie wholly before the window's first
    const int base = ci < nk ? ci * KC : (lo / KC + ci - nk) * KC;
    if (base > pos) return;
    const int group = n_heads / n_kv, h0 = g * group;
    extern __shared__ __align__(16) float sm[];
    float* qs = sm;                                     // [group][d]
    float* sc = qs + group * ((d + 3) & ~3);            // [group][KC] scores, then probabilities
    float* ml = sc + group * KC;                        // [group][2] maximum and sum
    int64_t* rowoff = reinterpret_cast<int64_t*>(ml + 2 * GMAX);   // [KC]
    const int dq = (d + 3) & ~3;
    for (int i = tid; i < group * d; i += KC) {
        const int gq = i / d, e = i - gq * d;
        qs[gq * dq + e] = ib::to_f32(q[(t * n_heads + h0 + gq) * d + e]);
    }
    __syncthreads();
    const int* table = block_table + int64_t(sg) * max_blocks;
    const int key = base + tid;
    const bool valid = key <= pos && (key >= lo || key < keep_end);
    // a key in the gap between the kept keys and the window takes the row of the chunk's first visible key (weight 0)
    const int first_seen = base < keep_end ? base : max(lo, base);
    const bool in_gap = !valid && key > first_seen && key < lo;
    float acc[GB];
#pragma unroll
    for (int gq = 0; gq < GB; gq++) acc[gq] = 0.0f;
    bool have = false;
    if (in_gap) {
        const int page = table[first_seen / page_size];
        rowoff[tid] = (page < 0 || page >= n_pages) ? 0 : (int64_t(page) * n_kv + g) * page_size + first_seen % page_size;
    } else if (valid) {
        const int page = table[key / page_size];
        if (page < 0 || page >= n_pages) {
            if (status) atomicExch(status, 3);
            rowoff[tid] = 0;
        } else {
            have = true;
            const int64_t row = (int64_t(page) * n_kv + g) * page_size + key % page_size;
            rowoff[tid] = row;
            const T* kr = k_cache + row * d;
            if (vec) {
                // four 16-byte loads of the row are in flight together (a thread's row is its own: nothing is shared)
                for (int e0 = 0; e0 < d; e0 += 32) {
                    float kv[4][8];
#pragma unroll
                    for (int b4 = 0; b4 < 4; b4++) {
                        if (e0 + 8 * b4 < d) load8<T>(kr + e0 + 8 * b4, kv[b4]);
                    }
#pragma unroll
                    for (int b4 = 0; b4 < 4; b4++) {
                        const int e = e0 + 8 * b4;
                        if (e < d) {
#pragma unroll
                            for (int gq = 0; gq < GB; gq++) {
                                if (gq < group) {
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
                }
            } else {
                for (int e = 0; e < d; e++) {
                    const float kv = ib::to_f32(kr[e]);
#pragma unroll
                    for (int gq = 0; gq < GB; gq++)
                        if (gq < group) acc[gq] = fmaf(qs[gq * dq + e], kv, acc[gq]);
                }
            }
        }
    } else {
        rowoff[tid] = 0;
    }
#pragma unroll
    for (int gq = 0; gq < GB; gq++) {
        if (gq < group) {
            float sv = -INFINITY;
            if (have) {
                sv = acc[gq] * scale;
                if (dist_bias) sv += dist_bias[int64_t(min(pos - key, bias_len - 1)) * n_heads + h0 + gq];
                if (slopes) sv = fmaf(-slopes[h0 + gq], float(pos - key), sv);
            }
            sc[gq * KC + tid] = sv;
        }
    }
    __syncthreads();
    for (int gq = warp; gq < group; gq += KC / 32) {
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
    const int j0 = first_seen - base, j1 = (ci < nk ? min(keep_end - 1, base + KC - 1) : min(pos, base + KC - 1)) - base;
    if (vec_v) {
        // Value rows reach shared memory VT keys at a time, by 16-byte loads that all threads issue together; then a
        // thread per channel adds them in ascending key order (the same order as the loop below).
        T* vt = reinterpret_cast<T*>(rowoff + KC);           // [VT][dv]
        constexpr int PER = 16 / int(sizeof(T));             // values per 16-byte load
        const int n_c = (dv + KC - 1) / KC;                  // channel passes of a thread (dv <= 2 KC)
        float o0[GB], o1[GB];
#pragma unroll
        for (int gq = 0; gq < GB; gq++) o0[gq] = o1[gq] = 0.0f;
        for (int js = j0; js <= j1; js += VT) {
            const int nj = min(VT, j1 - js + 1);
            const int per_row = dv / PER;
            __syncthreads();                                 // the last sub-tile has been read
            for (int i = tid; i < nj * per_row; i += KC) {
                const int jj = i / per_row, e = (i - jj * per_row) * PER;
                *reinterpret_cast<uint4*>(vt + jj * dv + e) = *reinterpret_cast<const uint4*>(v_cache + rowoff[js + jj] * dv + e);
            }
            __syncthreads();
            if (n_c > 1) {
                for (int jj = 0; jj < nj; jj++) {
                    const float va = tid < dv ? ib::to_f32(vt[jj * dv + tid]) : 0.0f;
                    const float vb = tid + KC < dv ? ib::to_f32(vt[jj * dv + tid + KC]) : 0.0f;
#pragma unroll
                    for (int gq = 0; gq < GB; gq++) {
                        if (gq < group) {
                            const float pj = sc[gq * KC + js + jj];
                            o0[gq] = fmaf(pj, va, o0[gq]);
                            o1[gq] = fmaf(pj, vb, o1[gq]);
                        }
                    }
                }
            } else {
#pragma unroll 4
                for (int jj = 0; jj < nj; jj++) {
                    const float va = tid < dv ? ib::to_f32(vt[jj * dv + tid]) : 0.0f;
#pragma unroll
                    for (int gq = 0; gq < GB; gq++)
                        if (gq < group) o0[gq] = fmaf(sc[gq * KC + js + jj], va, o0[gq]);
                }
            }
        }
#pragma unroll
        for (int gq = 0; gq < GB; gq++) {
            if (gq < group) {
                float* dst = parts + ((t * n_heads + h0 + gq) * n_chunks + ci) * int64_t(dv + 2) + 2;
                if (tid < dv) dst[tid] = o0[gq];
                if (tid + KC < dv) dst[tid + KC] = o1[gq];
            }
        }
    } else {
        for (int c = tid; c < dv; c += KC) {
            float o[GB];
#pragma unroll
            for (int gq = 0; gq < GB; gq++) o[gq] = 0.0f;
#pragma unroll 4
            for (int j = j0; j <= j1; j++) {
                const float vv = ib::to_f32(v_cache[rowoff[j] * dv + c]);
#pragma unroll
                for (int gq = 0; gq < GB; gq++)
                    if (gq < group) o[gq] = fmaf(sc[gq * KC + j], vv, o[gq]);
            }
#pragma unroll
            for (int gq = 0; gq < GB; gq++)
                if (gq < group) parts[((t * n_heads + h0 + gq) * n_chunks + ci) * int64_t(dv + 2) + 2 + c] = o[gq];
        }
    }
    if (tid < group) {
        float* dst = parts + ((t * n_heads + h0 + tid) * n_chunks + ci) * int64_t(dv + 2);
        dst[0] = ml[2 * tid];
        dst[1] = ml[2 * tid + 1];
    }
}

// One warp per (token, head): the chunks' parts in ascending order, the sink, the division; optionally times
// sigmoid(gate[t, gate_col + h dv + c]) (the logits of a gate per output channel, rows of leading dimension ldg).
template <typename T>
__global__ void split_attention_merge_kernel(const float* __restrict__ parts, const int* __restrict__ token_seg,
                                             const int* __restrict__ positions, const int* __restrict__ single_only,
                                             const float* __restrict__ sink, T* __restrict__ out, int64_t n_rows, int n_heads,
                                             int dv, int window, int n_chunks, int keep_first, const T* __restrict__ gate,
                                             int64_t ldg, int64_t gate_col) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t r = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int64_t t = r / n_heads;
    const int h = int(r - t * n_heads);
    const int sg = token_seg[t];
    if (single_only && single_only[sg + 1] - single_only[sg] > 1) return;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int nk = min((min(keep_first, lo) + KC - 1) / KC, lo / KC);
    const int n = min(n_chunks, nk + pos / KC - lo / KC + 1);
    const float* mine = parts + r * n_chunks * int64_t(dv + 2);
    const int64_t stride = dv + 2;
    // maxima and sums: a lane per chunk (in rounds of 32), then across the warp; every chunk's weight is computed once
    float m = sink ? sink[h] : -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, mine[i * stride]);
    m = ib::warp_max(m);
    float l = 0.0f;
    for (int i = lane; i < n; i += 32) l += mine[i * stride + 1] * expf(mine[i * stride] - m);
    l = ib::warp_sum(l) + (sink ? expf(sink[h] - m) : 0.0f);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    float acc[8];                                            // up to 256 channels a pass (8 per lane), chunks in ascending order
    for (int c0 = 0; c0 < dv; c0 += 256) {
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.0f;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const float w_mine = i0 + lane < n ? expf(mine[(i0 + lane) * stride] - m) : 0.0f;
            const int ni = min(32, n - i0);
            for (int i = 0; i < ni; i++) {
                const float w = __shfl_sync(0xffffffffu, w_mine, i);
                const float* row = mine + (i0 + i) * stride + 2 + c0;
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const int c = c0 + e * 32 + lane;
                    if (c < dv) acc[e] = fmaf(row[e * 32 + lane], w, acc[e]);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int c = c0 + e * 32 + lane;
            if (c >= dv) continue;
            const float o = acc[e];
        float y = o * inv;
        // (a gate per output channel: the result is rounded as the ungated kernel leaves it, then multiplied)
        if (gate) y = ib::to_f32(ib::from_f32<T>(y)) * sigmoid_(ib::to_f32(gate[t * ldg + gate_col + int64_t(h) * dv + c]));
        out[r * dv + c] = ib::from_f32<T>(y);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Decays of a linear attention whose key channels forget at learned, input-dependent rates:
//   z[t, c] = bias[c] + sum_r up[r, c] * low[t, r]      (low: the rows' columns [low_col, low_col + rank), float;
//                                                        up stored [rank, channels]: neighbouring threads, which
//                                                        are neighbouring channels, read neighbouring floats)
//   decay[t, c] = sigmoid(z) ^ (1 / tau) = exp(log_sigmoid(z) / tau)
// and, in the same pass, q[t, c] *= q_scale in place (columns [q_col, q_col + channels) of the rows).
__global__ void decay_gates_kernel(float* __restrict__ rows, int64_t ld, int q_col, int low_col, int rank,
                                   const float* __restrict__ up, const float* __restrict__ bias, float inv_tau, float q_scale,
                                   float* __restrict__ decay, int64_t n_tokens, int channels) {
    ib::pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_tokens * channels) return;
    const int64_t t = i / channels;
    const int c = int(i - t * channels);
    const float* low = rows + t * ld + low_col;
    float z = 0.0f;
    for (int r = 0; r < rank; r++) z = fmaf(up[int64_t(r) * channels + c], low[r], z);
    z += bias ? bias[c] : 0.0f;
    decay[i] = expf(log_sigmoid_(z) * inv_tau);
    rows[t * ld + q_col + c] *= q_scale;
}

// ------------------------------------------------------------------------------------------------
// Short causal filter per channel: y[t] = sum_j w[j][c] * u[t - (taps - 1) + j]; u before the segment's first row
// comes from the request's tail (its last taps - 1 inputs, oldest first; zeros for a new request). Weights tap-major.
__device__ __forceinline__ float filtered(const float* __restrict__ rows, int64_t ld, int64_t t, int i_local, int col,
                                          const float* __restrict__ w, int64_t w_stride, int taps,
                                          const float* __restrict__ tail, int64_t tail_ld) {
    if (taps <= 0 || !w) return rows[t * ld + col];
    float y = 0.0f;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;
        const float u = i_local >= back ? rows[(t - back) * ld + col] : tail[int64_t(taps - 1 + i_local - back) * tail_ld];
        y = fmaf(w[j * w_stride], u, y);
    }
    return y;
}

// What the gated delta rule reads, from the projected rows (float): raw columns from col0 are [q (G heads of d) |
// k (G x d) | v (H heads of dv)], each channel through its causal filter and silu; q and k of a head divided by
// sqrt(sum(x^2) + unit_eps), q also times q_scale; per head h: beta = sigmoid(raw[b_col + h]),
// g = exp(-exp(a_log[h]) * softplus(raw[a_col + h] + dt_bias[h])).
// prep rows (float, ldp): [q | k | v | g (H) | beta (H) | k.q (G)].
// One warp per (token, unit): G units of a (q, k) head pair, H units of a v head, one unit for the heads' scalars.
constexpr int PREP_PER_LANE = 8;         // heads of up to 32 * PREP_PER_LANE channels

// The newest input of channel c joins its request's tail, the oldest leaves (steps of one token per request: the lane
// that filtered the channel is the tail's only reader).
__device__ __forceinline__ void shift_tail(float* tail, int64_t channels, int taps, int c, float newest) {
    for (int idx = 0; idx + 1 < taps - 1; idx++) tail[int64_t(idx) * channels + c] = tail[int64_t(idx + 1) * channels + c];
    tail[int64_t(taps - 2) * channels + c] = newest;
}

__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ rows, int64_t ld, int col0, int a_col, int b_col,
                     const float* __restrict__ filt_w, int taps, float* tails, int inline_tail,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, float unit_eps, float q_scale,
                     const int* __restrict__ token_seg, const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                     float* __restrict__ prep, int64_t ldp, int64_t n_tokens, int n_heads, int n_qk, int d, int dv) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int units = n_qk + n_heads + 1;
    const int64_t wi = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wi >= n_tokens * units) return;
    const int64_t t = wi / units;
    const int u = int(wi - t * units);
    const int channels = 2 * n_qk * d + n_heads * dv;
    const int s = token_seg[t];
    const int i_local = int(t - seg_start[s]);
    float* tail = taps > 1 ? tails + (int64_t(seg_slot[s]) * (taps - 1)) * channels : nullptr;
    const bool move = inline_tail && taps > 1;
    float* out = prep + t * ldp;
    const int g_off = 2 * n_qk * d + n_heads * dv;
    if (u < n_qk) {
        float qv[PREP_PER_LANE], kv[PREP_PER_LANE];
        float sq = 0.0f, sk = 0.0f, dot = 0.0f;
#pragma unroll
        for (int r = 0; r < PREP_PER_LANE; r++) {
            const int j = lane + 32 * r;
            qv[r] = kv[r] = 0.0f;
            if (j < d) {
                const int cq = u * d + j, ck = n_qk * d + u * d + j;
                qv[r] = silu_(filtered(rows, ld, t, i_local, col0 + cq, filt_w + cq, channels, taps, tail + cq, channels));
                kv[r] = silu_(filtered(rows, ld, t, i_local, col0 + ck, filt_w + ck, channels, taps, tail + ck, channels));
                if (move) {
                    shift_tail(tail, channels, taps, cq, rows[t * ld + col0 + cq]);
                    shift_tail(tail, channels, taps, ck, rows[t * ld + col0 + ck]);
                }
                sq = fmaf(qv[r], qv[r], sq);
                sk = fmaf(kv[r], kv[r], sk);
                dot = fmaf(qv[r], kv[r], dot);
            }
        }
        sq = ib::warp_sum(sq);
        sk = ib::warp_sum(sk);
        dot = ib::warp_sum(dot);
        const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
#pragma unroll
        for (int r = 0; r < PREP_PER_LANE; r++) {
            const int j = lane + 32 * r;
            if (j < d) {
                out[u * d + j] = qv[r] * fq;
                out[n_qk * d + u * d + j] = kv[r] * fk;
            }
        }
        if (lane == 0) out[g_off + 2 * n_heads + u] = dot * fq * fk;
    } else if (u < n_qk + n_heads) {
        const int h = u - n_qk;
        for (int j = lane; j < dv; j += 32) {
            const int c = 2 * n_qk * d + h * dv + j;
            out[c] = silu_(filtered(rows, ld, t, i_local, col0 + c, filt_w + c, channels, taps, tail + c, channels));
            if (move) shift_tail(tail, channels, taps, c, rows[t * ld + col0 + c]);
        }
    } else {
        for (int h = lane; h < n_heads; h += 32) {
            const float a = rows[t * ld + a_col + h], b = rows[t * ld + b_col + h];
            out[g_off + h] = expf(-expf(a_log[h]) * softplus_(a + dt_bias[h]));
            out[g_off + n_heads + h] = sigmoid_(b);
        }
    }
}

// After a step: the tail of every segment's request becomes the last taps - 1 values of (old tail, the step's rows).
// One thread per (segment, channel) moves its values oldest first, reading ahead of what it writes.
__global__ void tail_update_kernel(const float* __restrict__ rows, int64_t ld, int col0, int channels, int taps,
                                   float* __restrict__ tails, const int* __restrict__ seg_start,
                                   const int* __restrict__ seg_slot) {
    ib::pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= channels) return;
    const int keep = taps - 1;
    const int64_t t0 = seg_start[s];
    const int len = int(seg_start[s + 1] - t0);
    float* tail = tails + (int64_t(seg_slot[s]) * keep) * channels + c;
    for (int idx = 0; idx < keep; idx++) {
        const int src = len - keep + idx;
        tail[int64_t(idx) * channels] = src >= 0 ? rows[(t0 + src) * ld + col0 + c] : tail[int64_t(idx + len) * channels];
    }
}

// ------------------------------------------------------------------------------------------------
// Linear recurrences with a matrix state S [d, dv] per head (float, kept in `state` between steps), over the tokens of
// every segment in order:
//   MODE 0 (a decay per key channel):  S <- diag(a_t) S + k_t v_t^T;               o_t = S^T q_t
//   MODE 1 (gated delta rule):         S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//   MODE 2 (a constant decay per head):  S <- g S + k_t v_t^T;                       o_t = S^T q_t
//   MODE 3 (a decay per key channel, a bonus for the current token):
//                                       o_t = (S + diag(u) k_t v_t^T)^T q_t;  then  S <- diag(a_t) S + k_t v_t^T
// MODE 1 is computed from the old state in one sweep: r = S^T k, p = S^T q, u = beta (v - g r), o = g p + u (k.q),
// S <- g S + k u^T, with k.q given per token (aux rows). MODE 2 reads g at aux_col + h of the token's aux row (a
// leading dimension of 0: one row for every token). MODE 3 reads its decays as MODE 0 and u [heads, d] from `bonus`.
// A column of S belongs to LK = 8 neighbouring lanes, lane j of them keeping rows j R .. j R + R - 1 in registers
// (R >= d / 8, rows beyond d are zero and stay zero); a warp has 4 columns, a CTA `cb` columns of one (segment, head).
// Column sums are added within a lane in four chains and across the 8 lanes by shuffles, in an order that depends on
// (d, dv) only; tokens are staged `chunk` at a time in shared memory, and no thread waits for another CTA.
// q and k of head h are those of head h / heads_per_qk (MODE 1: several value heads share a (q, k) head).
// Inputs are float rows: q, k, v in `rows` (ld); MODE 0: decay in `aux` at aux_col + h d; MODE 1: g at aux_col + h,
// beta at aux_col + H + h, k.q at aux_col + 2 H + h / heads_per_qk. raw_out [tokens, H, dv] float.
constexpr int LK = 8;

__device__ __forceinline__ void copy_async16(float* smem_dst, const float* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copy_async4(float* smem_dst, const float* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(uint32_t(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src) : "memory");
}

// One token's operands of a thread: its R rows of q, k (and of the decays), the value of its column, the scalars.
template <int R, int MODE>
struct ScanOperands {
    float4 q[R / 4], k[R / 4], a[(MODE == 0 || MODE == 3) ? R / 4 : 1];
    float v, g, beta, kq;
    __device__ __forceinline__ void load(const float* qs, const float* ks, const float* as, const float* vs, int c, int dpp, int off,
                                         int cb, int col_l) {
        const float4* q4 = reinterpret_cast<const float4*>(qs + c * dpp + off);
        const float4* k4 = reinterpret_cast<const float4*>(ks + c * dpp + off);
#pragma unroll
        for (int i = 0; i < R / 4; i++) { q[i] = q4[i]; k[i] = k4[i]; }
        if (MODE == 0 || MODE == 3) {
            const float4* a4 = reinterpret_cast<const float4*>(as + c * dpp + off);
#pragma unroll
            for (int i = 0; i < R / 4; i++) a[i] = a4[i];
        } else {
            g = as[c * 4 + 0]; beta = as[c * 4 + 1]; kq = as[c * 4 + 2];
        }
        v = vs[c * cb + col_l];
    }
};

// One token through a thread's share of the state; returns the column's read-out (valid in every lane of its group).
template <int R, int MODE>
__device__ __forceinline__ float scan_token(float (&S)[R], const ScanOperands<R, MODE>& x, const float* U) {
    const float v = x.v;
    if (MODE == 2) {
        const float g = x.g;
        float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
        for (int i4 = 0; i4 < R / 4; i4++) {
            const float4 k = x.k[i4], q = x.q[i4];
            S[4 * i4 + 0] = fmaf(g, S[4 * i4 + 0], k.x * v);
            S[4 * i4 + 1] = fmaf(g, S[4 * i4 + 1], k.y * v);
            S[4 * i4 + 2] = fmaf(g, S[4 * i4 + 2], k.z * v);
            S[4 * i4 + 3] = fmaf(g, S[4 * i4 + 3], k.w * v);
            p0 = fmaf(S[4 * i4 + 0], q.x, p0);
            p1 = fmaf(S[4 * i4 + 1], q.y, p1);
            p2 = fmaf(S[4 * i4 + 2], q.z, p2);
            p3 = fmaf(S[4 * i4 + 3], q.w, p3);
        }
        float p = (p0 + p1) + (p2 + p3);
        p += __shfl_xor_sync(0xffffffffu, p, 1);
        p += __shfl_xor_sync(0xffffffffu, p, 2);
        p += __shfl_xor_sync(0xffffffffu, p, 4);
        return p;
    }
    if (MODE == 3) {
        float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
        for (int i4 = 0; i4 < R / 4; i4++) {
            const float4 a = x.a[i4], k = x.k[i4], q = x.q[i4];
            const float w0 = k.x * v, w1 = k.y * v, w2 = k.z * v, w3 = k.w * v;
            p0 = fmaf(fmaf(U[4 * i4 + 0], w0, S[4 * i4 + 0]), q.x, p0);
            p1 = fmaf(fmaf(U[4 * i4 + 1], w1, S[4 * i4 + 1]), q.y, p1);
            p2 = fmaf(fmaf(U[4 * i4 + 2], w2, S[4 * i4 + 2]), q.z, p2);
            p3 = fmaf(fmaf(U[4 * i4 + 3], w3, S[4 * i4 + 3]), q.w, p3);
            S[4 * i4 + 0] = fmaf(a.x, S[4 * i4 + 0], w0);
            S[4 * i4 + 1] = fmaf(a.y, S[4 * i4 + 1], w1);
            S[4 * i4 + 2] = fmaf(a.z, S[4 * i4 + 2], w2);
            S[4 * i4 + 3] = fmaf(a.w, S[4 * i4 + 3], w3);
        }
        float p = (p0 + p1) + (p2 + p3);
        p += __shfl_xor_sync(0xffffffffu, p, 1);
        p += __shfl_xor_sync(0xffffffffu, p, 2);
        p += __shfl_xor_sync(0xffffffffu, p, 4);
        return p;
    }
    if (MODE == 0) {
        float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
        for (int i4 = 0; i4 < R / 4; i4++) {
            const float4 a = x.a[i4], k = x.k[i4], q = x.q[i4];
            S[4 * i4 + 0] = fmaf(a.x, S[4 * i4 + 0], k.x * v);
            S[4 * i4 + 1] = fmaf(a.y, S[4 * i4 + 1], k.y * v);
            S[4 * i4 + 2] = fmaf(a.z, S[4 * i4 + 2], k.z * v);
            S[4 * i4 + 3] = fmaf(a.w, S[4 * i4 + 3], k.w * v);
            p0 = fmaf(S[4 * i4 + 0], q.x, p0);
            p1 = fmaf(S[4 * i4 + 1], q.y, p1);
            p2 = fmaf(S[4 * i4 + 2], q.z, p2);
            p3 = fmaf(S[4 * i4 + 3], q.w, p3);
        }
        float p = (p0 + p1) + (p2 + p3);
        p += __shfl_xor_sync(0xffffffffu, p, 1);
        p += __shfl_xor_sync(0xffffffffu, p, 2);
        p += __shfl_xor_sync(0xffffffffu, p, 4);
        return p;
    }
    const float g = x.g;
    float r0 = 0.0f, r1 = 0.0f, p0 = 0.0f, p1 = 0.0f;
#pragma unroll
    for (int i4 = 0; i4 < R / 4; i4++) {
        const float4 k = x.k[i4], q = x.q[i4];
        r0 = fmaf(S[4 * i4 + 0], k.x, r0);
        r1 = fmaf(S[4 * i4 + 1], k.y, r1);
        r0 = fmaf(S[4 * i4 + 2], k.z, r0);
        r1 = fmaf(S[4 * i4 + 3], k.w, r1);
        p0 = fmaf(S[4 * i4 + 0], q.x, p0);
        p1 = fmaf(S[4 * i4 + 1], q.y, p1);
        p0 = fmaf(S[4 * i4 + 2], q.z, p0);
        p1 = fmaf(S[4 * i4 + 3], q.w, p1);
    }
    float r = r0 + r1, p = p0 + p1;
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    p += __shfl_xor_sync(0xffffffffu, p, 1);
    r += __shfl_xor_sync(0xffffffffu, r, 2);
    p += __shfl_xor_sync(0xffffffffu, p, 2);
    r += __shfl_xor_sync(0xffffffffu, r, 4);
    p += __shfl_xor_sync(0xffffffffu, p, 4);
    const float u = x.beta * (v - g * r);
#pragma unroll
    for (int i4 = 0; i4 < R / 4; i4++) {
        const float4 k = x.k[i4];
        S[4 * i4 + 0] = fmaf(k.x, u, g * S[4 * i4 + 0]);
        S[4 * i4 + 1] = fmaf(k.y, u, g * S[4 * i4 + 1]);
        S[4 * i4 + 2] = fmaf(k.z, u, g * S[4 * i4 + 2]);
        S[4 * i4 + 3] = fmaf(k.w, u, g * S[4 * i4 + 3]);
    }
    return fmaf(u, x.kq, g * p);
}

// Staging: a token's q, k (and decays) lie in shared memory as [lane group][R + 4] (the four floats of padding keep
// the eight lanes' 16-byte loads on different banks), rows beyond d zero. With `pipelined` (every row, column offset
// and size a multiple of four floats) the rows are copied as they lie by asynchronous 16-byte copies, one chunk ahead
// of the one being computed; otherwise element by element. The operands of token c + 1 are read into registers while
// token c is computed. The arithmetic per token is the same in every case.
template <int R, int MODE>
__global__ void __launch_bounds__(256)
state_scan_kernel(const float* __restrict__ rows, int64_t ld, int q_col, int k_col, int v_col,
                  const float* __restrict__ aux, int64_t lda, int aux_col, float* __restrict__ state,
                  const int* __restrict__ seg_start, const int* __restrict__ seg_slot, float* __restrict__ raw_out,
                  int n_heads, int heads_per_qk, int d, int dv, int cb, int chunk, int write_state, int pipelined,
                  const float* __restrict__ bonus, int act) {
    extern __shared__ __align__(16) float sm[];
    constexpr int RP = R + 4, DPP = LK * RP;
    constexpr bool ROWS = MODE == 0 || MODE == 3;      // the decays are rows like q and k
    constexpr int N_SCAL = MODE == 1 ? 3 : 1;          // scalars per token otherwise
    const int n_buf = pipelined ? 2 : 1;
    const int a_tok = ROWS ? DPP : 4;
    float* qs = sm;                          // [n_buf][chunk][DPP]
    float* ks = qs + n_buf * chunk * DPP;
    float* as = ks + n_buf * chunk * DPP;    // MODE 0: [n_buf][chunk][DPP] decays; MODE 1: [n_buf][chunk][4] g, beta, k.q
    float* vs = as + n_buf * chunk * a_tok;  // [n_buf][chunk][cb]
    const int total = n_buf * chunk * (2 * DPP + a_tok + cb);
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int hq = h / heads_per_qk;
    const int lk = tid & (LK - 1), col_l = tid >> 3;
    const int col0 = blockIdx.z * cb, col = col0 + col_l;
    const bool live = col < dv;
    const int k0 = lk * R, off = lk * RP;
    for (int i = tid; i < total; i += blockDim.x) sm[i] = 0.0f;       // padding and rows beyond d stay zero
    ib::pdl_wait();
    const int64_t t0 = seg_start[s];
    const int len = int(seg_start[s + 1] - t0);
    float* S_g = state + (int64_t(seg_slot[s]) * n_heads + h) * int64_t(d) * dv;
    float S[R];
#pragma unroll
    for (int i = 0; i < R; i++) S[i] = (live && k0 + i < d) ? S_g[int64_t(k0 + i) * dv + col] : 0.0f;
    float U[MODE == 3 ? R : 1];
    if (MODE == 3) {
#pragma unroll
        for (int i = 0; i < R; i++) U[i] = k0 + i < d ? bonus[int64_t(h) * d + k0 + i] : 0.0f;
    }
    __syncthreads();

    auto request = [&](int c0, int b) {      // asynchronous copies of the chunk that starts at token c0 into buffer b
        const int n = min(chunk, len - c0);
        const int d4 = d / 4, cb4 = cb / 4;
        for (int idx = tid; idx < n * d4; idx += blockDim.x) {
            const int c = idx / d4, j = (idx - c * d4) * 4;
            const int dst = (b * chunk + c) * DPP + (j / R) * RP + j % R;
            const float* row = rows + (t0 + c0 + c) * ld;
            copy_async16(qs + dst, row + q_col + hq * d + j);
            copy_async16(ks + dst, row + k_col + hq * d + j);
            if (ROWS) copy_async16(as + dst, aux + (t0 + c0 + c) * lda + aux_col + h * d + j);
        }
        if (!ROWS) {
            for (int idx = tid; idx < n * N_SCAL; idx += blockDim.x) {
                const int c = idx / N_SCAL, e = idx - c * N_SCAL;
                const float* ar = aux + (t0 + c0 + c) * lda + aux_col;
                copy_async4(as + (b * chunk + c) * 4 + e, ar + (e == 0 ? h : (e == 1 ? n_heads + h : 2 * n_heads + hq)));
            }
        }
        for (int idx = tid; idx < n * cb4; idx += blockDim.x) {
            const int c = idx / cb4, j = (idx - c * cb4) * 4;
            if (col0 + j < dv) copy_async16(vs + (b * chunk + c) * cb + j, rows + (t0 + c0 + c) * ld + v_col + h * dv + col0 + j);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto stage = [&](int c0) {               // the same chunk element by element (any sizes and offsets)
        const int n = min(chunk, len - c0);
        for (int idx = tid; idx < n * d; idx += blockDim.x) {
            const int c = idx / d, j = idx - c * d;
            const int dst = c * DPP + (j / R) * RP + j % R;
            const float* row = rows + (t0 + c0 + c) * ld;
            qs[dst] = act ? silu_(row[q_col + hq * d + j]) : row[q_col + hq * d + j];
            ks[dst] = act ? silu_(row[k_col + hq * d + j]) : row[k_col + hq * d + j];
            if (ROWS) as[dst] = aux[(t0 + c0 + c) * lda + aux_col + h * d + j];
        }
        if (!ROWS) {
            for (int c = tid; c < n; c += blockDim.x) {
                const float* ar = aux + (t0 + c0 + c) * lda + aux_col;
                as[c * 4 + 0] = ar[h];
                if (MODE == 1) {
                    as[c * 4 + 1] = ar[n_heads + h];
                    as[c * 4 + 2] = ar[2 * n_heads + hq];
                }
            }
        }
        for (int idx = tid; idx < n * cb; idx += blockDim.x) {
            const int c = idx / cb, j = col0 + (idx - c * cb);
            const float vv = j < dv ? rows[(t0 + c0 + c) * ld + v_col + h * dv + j] : 0.0f;
            vs[idx] = act ? silu_(vv) : vv;
        }
    };

    if (pipelined && len > 0) request(0, 0);
    int b = 0;
    for (int c0 = 0; c0 < len; c0 += chunk) {
        const int n = min(chunk, len - c0);
        if (pipelined) {
            if (c0 + chunk < len) {
                request(c0 + chunk, b ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        } else {
            stage(c0);
        }
        __syncthreads();                     // the chunk has arrived
        const float* qb = qs + b * chunk * DPP;
        const float* kb = ks + b * chunk * DPP;
        const float* ab = as + b * chunk * a_tok;
        const float* vb = vs + b * chunk * cb;
        ScanOperands<R, MODE> cur, nxt;
        cur.load(qb, kb, ab, vb, 0, DPP, off, cb, col_l);
        for (int c = 0; c < n; c++) {
            if (c + 1 < n) nxt.load(qb, kb, ab, vb, c + 1, DPP, off, cb, col_l);
            const float o = scan_token<R, MODE>(S, cur, U);
            if (lk == 0 && live) raw_out[((t0 + c0 + c) * n_heads + h) * int64_t(dv) + col] = o;
            cur = nxt;
        }
        __syncthreads();                     // every thread has read this buffer: the copies after next may fill it
        if (pipelined) b ^= 1;
    }
    if (write_state && live) {
#pragma unroll
        for (int i = 0; i < R; i++)
            if (k0 + i < d) S_g[int64_t(k0 + i) * dv + col] = S[i];
    }
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * w [* silu(gate)], lanes striding over the columns; the
// gate's logits are columns gate_col + h dv + j of rows `gate` (leading dimension ldg).
template <typename TG, typename TOut>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                      const TG* __restrict__ gate, int64_t ldg, int gate_col, TOut* __restrict__ out,
                                      int64_t n_rows, int n_heads, int dv) {
    ib::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t r = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int64_t t = r / n_heads;
    const int h = int(r - t * n_heads);
    const float* x = o + r * dv;
    float ss = 0.0f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(x[j], x[j], ss);
    ss = ib::warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / float(dv) + eps);
    for (int j = lane; j < dv; j += 32) {
        float y = x[j] * f * w[j];
        if (gate) y *= silu_(ib::to_f32(gate[t * ldg + gate_col + h * dv + j]));
        out[r * dv + j] = ib::from_f32<TOut>(y);
    }
}

}  // namespace

// ================================================================================================
// C entry points. dtype arguments: 0 = float, 1 = bfloat16.

IB_EXPORT int ib_norm_add(const float* x, const float* y, const float* w, float eps, float* out, void* copy, int copy_dtype,
                          int64_t n_tokens, int64_t width, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return IB_OK;
    if (!y || !w || !out) return ib::fail(IB_ERR_ARG, "ib_norm_add: rows, weight and result are needed");
    if (copy && copy_dtype == IB_BF16)
        IB_LAUNCH(norm_add_kernel<bf16>, unsigned(n_tokens), 256, 0, x, y, w, eps, out, (bf16*)copy, width);
    else if (!copy || copy_dtype == IB_F32)
        IB_LAUNCH(norm_add_kernel<float>, unsigned(n_tokens), 256, 0, x, y, w, eps, out, (float*)copy, width);
    else
        return ib::fail(IB_ERR_ARG, "ib_norm_add: unknown dtype %d", copy_dtype);
    return ib::check_launch("ib_norm_add");
}

IB_EXPORT int ib_cast_rows(const float* x, void* out, int dtype, int64_t n, cudaStream_t stream) {
    if (n <= 0) return IB_OK;
    if (dtype != IB_BF16) return ib::fail(IB_ERR_ARG, "ib_cast_rows: unknown dtype %d", dtype);
    IB_LAUNCH(cast_rows_kernel<bf16>, blocks_for(n, 256), 256, 0, x, (bf16*)out, n);
    return ib::check_launch("ib_cast_rows");
}

IB_EXPORT int ib_dual_norm_sum(const float* a, const float* wa, float sa, const float* b, const float* wb, float sb, float eps,
                               const float* x, const float* wo, float eps_o, float* out, void* copy, int copy_dtype,
                               int64_t n_tokens, int64_t width, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return IB_OK;
    if (!a || !b || !wa || !wb || !out) return ib::fail(IB_ERR_ARG, "ib_dual_norm_sum: two terms with their weights are needed");
    const size_t smem = size_t(width) * sizeof(float);
    if (smem > 48 * 1024) return ib::fail(IB_ERR_ARG, "ib_dual_norm_sum: rows of %lld floats do not fit", (long long)width);
    if (copy && copy_dtype == IB_BF16)
        IB_LAUNCH(dual_norm_sum_kernel<bf16>, unsigned(n_tokens), 256, smem, a, wa, sa, b, wb, sb, eps, x, wo, eps_o, out, (bf16*)copy, width);
    else if (!copy || copy_dtype == IB_F32)
        IB_LAUNCH(dual_norm_sum_kernel<float>, unsigned(n_tokens), 256, smem, a, wa, sa, b, wb, sb, eps, x, wo, eps_o, out, (float*)copy, width);
    else
        return ib::fail(IB_ERR_ARG, "ib_dual_norm_sum: unknown dtype %d", copy_dtype);
    return ib::check_launch("ib_dual_norm_sum");
}

IB_EXPORT int ib_glu_act(const void* rows, int64_t ld, int64_t gate_col, int64_t up_col, int64_t width, int kind, float limit,
                         float limit2, float slope, const float* scale, int64_t group, int64_t n_groups, void* out,
                         int64_t n_tokens, int dtype, cudaStream_t stream) {
    const int64_t n = n_tokens * width;
    if (n <= 0) return IB_OK;
    if (kind < 0 || kind > 2) return ib::fail(IB_ERR_ARG, "ib_glu_act: unknown activation %d", kind);
    if (dtype == IB_F32)
        IB_LAUNCH(glu_act_kernel<float>, blocks_for(n, 256), 256, 0, (const float*)rows, ld, gate_col, up_col, width, kind, limit,
                  limit2, slope, scale, group, n_groups, (float*)out, n);
    else if (dtype == IB_BF16 && width % 8 == 0 && ld % 8 == 0 && gate_col % 8 == 0 && up_col % 8 == 0 && group % 8 == 0 &&
             !((uintptr_t(rows) | uintptr_t(out)) & 15))
        // (chosen by sizes and addresses, never by the number of rows)
        IB_LAUNCH(glu_act_vec_kernel, blocks_for(n / 8, 256), 256, 0, (const bf16*)rows, ld, gate_col, up_col, width / 8, kind, limit,
                  limit2, slope, scale, group, n_groups, (bf16*)out, n / 8);
    else if (dtype == IB_BF16)
        IB_LAUNCH(glu_act_kernel<bf16>, blocks_for(n, 256), 256, 0, (const bf16*)rows, ld, gate_col, up_col, width, kind, limit,
                  limit2, slope, scale, group, n_groups, (bf16*)out, n);
    else
        return ib::fail(IB_ERR_ARG, "ib_glu_act: unknown dtype %d", dtype);
    return ib::check_launch("ib_glu_act");
}

IB_EXPORT int ib_route(const float* logits, int64_t n_tokens, int n_experts, int top, int n_groups, int keep, float sum_eps,
                       float* weights, int* chosen, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_experts <= 0 || n_groups <= 0 || n_experts % n_groups || keep <= 0 || keep > n_groups || top <= 0 ||
        top > keep * (n_experts / n_groups))
        return ib::fail(IB_ERR_ARG, "ib_route: %d experts in %d groups, %d kept, %d chosen", n_experts, n_groups, keep, top);
    const size_t smem = size_t(4) * (n_experts + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return ib::fail(IB_ERR_ARG, "ib_route: %d experts do not fit", n_experts);
    IB_LAUNCH(route_kernel, blocks_for(n_tokens, 4), 128, smem, logits, n_tokens, n_experts, top, n_groups, keep, sum_eps, weights, chosen);
    return ib::check_launch("ib_route");
}

IB_EXPORT int ib_rownorm_store(const void* rows, int64_t ld, int col0, const float* wq, const float* wk, float eps,
                               const int* positions, const int* token_seg, const int* block_table, int64_t max_blocks,
                               void* q_out, void* k_cache, void* v_cache, int64_t n_tokens, int n_heads, int n_kv, int d, int dv,
                               int page_size, int write_cache, int64_t n_pages, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv <= 0 || d <= 0 || dv <= 0 || page_size <= 0) return ib::fail(IB_ERR_ARG, "ib_rownorm_store: bad sizes");
    if (dtype == IB_F32)
        IB_LAUNCH(rownorm_store_kernel<float>, unsigned(n_tokens), 256, 0, (const float*)rows, ld, col0, wq, wk, eps, positions, token_seg,
                  block_table, max_blocks, (float*)q_out, (float*)k_cache, (float*)v_cache, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status);
    else if (dtype == IB_BF16)
        IB_LAUNCH(rownorm_store_kernel<bf16>, unsigned(n_tokens), 256, 0, (const bf16*)rows, ld, col0, wq, wk, eps, positions, token_seg,
                  block_table, max_blocks, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, n_heads, n_kv, d, dv, page_size, write_cache, n_pages, status);
    else
        return ib::fail(IB_ERR_ARG, "ib_rownorm_store: unknown dtype %d", dtype);
    return ib::check_launch("ib_rownorm_store");
}

// Floats of workspace that ib_attention_split needs for n_tokens tokens whose queries see up to `visible` keys.
IB_EXPORT int64_t ib_attention_split_workspace(int64_t n_tokens, int n_heads, int dv, int visible, int keep_first) {
    const int64_t n_chunks = (visible + KC - 1) / KC + 1 + (keep_first > 0 ? (keep_first + KC - 1) / KC : 0);
    return n_tokens * n_heads * n_chunks * (dv + 2);
}

// q, out [tokens, heads * d / dv]; caches [pages, kv heads, page_size, d / dv]; `visible`: the most keys a query of the
// step sees (its window, or the longest context); workspace as ib_attention_split_workspace says.
IB_EXPORT int ib_attention_split(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int64_t max_blocks,
                                 const int* token_seg, const int* positions, const int* single_only, void* out, float* workspace,
                                 int64_t n_tokens, int n_heads, int n_kv, int d, int dv, int page_size, int window, float scale,
                                 int64_t n_pages, const float* dist_bias, int bias_len, const float* sink, int visible, int dtype,
                                 int* status, cudaStream_t stream, int keep_first, const float* slopes, const void* gate, int64_t ldg,
                                 int64_t gate_col) {
    if (n_tokens <= 0) return IB_OK;
    if (n_kv <= 0 || n_heads % n_kv || n_heads / n_kv > GMAX)
        return ib::fail(IB_ERR_ARG, "ib_attention_split: %d heads on %d kv heads (groups of up to %d)", n_heads, n_kv, GMAX);
    if (d <= 0 || dv <= 0 || d > 512 || dv > 1024 || page_size <= 0 || visible <= 0 || !workspace)
        return ib::fail(IB_ERR_ARG, "ib_attention_split: bad sizes");
    if (dist_bias && bias_len <= 0) return ib::fail(IB_ERR_ARG, "ib_attention_split: a distance bias needs at least one row");
    if (keep_first < 0 || (keep_first > 0 && window <= 0)) keep_first = 0;     // without a window every key is seen anyway
    const int n_chunks = (visible + KC - 1) / KC + 1 + (keep_first > 0 ? (keep_first + KC - 1) / KC : 0);
    if (n_kv > 65535 || n_chunks > 65535) return ib::fail(IB_ERR_ARG, "ib_attention_split: too many kv heads or chunks");
    const int group = n_heads / n_kv;
    const size_t item = dtype == IB_F32 ? 4 : 2;
    size_t smem = size_t(group * ((d + 3) & ~3) + group * KC + 2 * GMAX) * sizeof(float) + KC * sizeof(int64_t);
    // values through shared memory where a row is whole 16-byte pieces and at most two channels fall to a thread
    const int vec_v = (dv * item) % 16 == 0 && dv <= 2 * KC && !(uintptr_t(v_cache) & 15) && smem + size_t(VT) * dv * item <= 48 * 1024;
    if (vec_v) smem += size_t(VT) * dv * item;
    if (smem > 48 * 1024) return ib::fail(IB_ERR_ARG, "ib_attention_split: %d heads of %d do not fit", group, d);
    const dim3 grid{unsigned(n_tokens), unsigned(n_kv), unsigned(n_chunks)};
    const int64_t rows = n_tokens * n_heads;
    const int vec = d % 8 == 0 && !(uintptr_t(k_cache) & 15);
    const int gb = group <= 1 ? 1 : (group <= 2 ? 2 : (group <= 4 ? 4 : (group <= 8 ? 8 : 16)));
#define IB_SPLIT(TT, GG)                                                                                                          \
    IB_LAUNCH((split_attention_kernel<TT, GG>), grid, KC, smem, (const TT*)q, (const TT*)k_cache, (const TT*)v_cache, block_table, \
              max_blocks, token_seg, positions, single_only, workspace, n_heads, n_kv, d, dv, page_size, window, scale, n_pages,  \
              dist_bias, bias_len, n_chunks, vec, vec_v, status, keep_first, slopes)
#define IB_SPLIT_BY_GROUP(TT)                                                                                                     \
    do {                                                                                                                          \
        if (gb == 1) IB_SPLIT(TT, 1); else if (gb == 2) IB_SPLIT(TT, 2); else if (gb == 4) IB_SPLIT(TT, 4);                       \
        else if (gb == 8) IB_SPLIT(TT, 8); else IB_SPLIT(TT, 16);                                                                 \
    } while (0)
    if (dtype == IB_F32) {
        IB_SPLIT_BY_GROUP(float);
        IB_LAUNCH(split_attention_merge_kernel<float>, blocks_for(rows, 4), 128, 0, workspace, token_seg, positions, single_only, sink,
                  (float*)out, rows, n_heads, dv, window, n_chunks, keep_first, (const float*)gate, ldg, gate_col);
    } else if (dtype == IB_BF16) {
        IB_SPLIT_BY_GROUP(bf16);
        IB_LAUNCH(split_attention_merge_kernel<bf16>, blocks_for(rows, 4), 128, 0, workspace, token_seg, positions, single_only, sink,
                  (bf16*)out, rows, n_heads, dv, window, n_chunks, keep_first, (const bf16*)gate, ldg, gate_col);
    } else {
        return ib::fail(IB_ERR_ARG, "ib_attention_split: unknown dtype %d", dtype);
    }
#undef IB_SPLIT_BY_GROUP
#undef IB_SPLIT
    return ib::check_launch("ib_attention_split");
}

IB_EXPORT int ib_decay_gates(float* rows, int64_t ld, int q_col, int low_col, int rank, const float* up, const float* bias,
                             float tau, float q_scale, float* decay, int64_t n_tokens, int channels, cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return IB_OK;
    if (rank <= 0 || !(tau > 0.0f)) return ib::fail(IB_ERR_ARG, "ib_decay_gates: rank %d, tau %f", rank, double(tau));
    IB_LAUNCH(decay_gates_kernel, blocks_for(n_tokens * channels, 256), 256, 0, rows, ld, q_col, low_col, rank, up, bias, 1.0f / tau,
              q_scale, decay, n_tokens, channels);
    return ib::check_launch("ib_decay_gates");
}

// The widest (q, k) head that ib_delta_prepare takes.
IB_EXPORT int ib_delta_prepare_max_dim() { return 32 * PREP_PER_LANE; }

// inline_tail (only for steps of one token per request): the kernel also moves the tails.
IB_EXPORT int ib_delta_prepare(const float* rows, int64_t ld, int col0, int a_col, int b_col, const float* filt_w, int taps,
                               float* tails, int inline_tail, const float* a_log, const float* dt_bias, float unit_eps, float q_scale,
                               const int* token_seg, const int* seg_start, const int* seg_slot, float* prep, int64_t ldp,
                               int64_t n_tokens, int n_heads, int n_qk, int d, int dv, cudaStream_t stream) {
    if (n_tokens <= 0) return IB_OK;
    if (n_heads <= 0 || n_qk <= 0 || n_heads % n_qk || d <= 0 || dv <= 0 || d > 32 * PREP_PER_LANE)
        return ib::fail(IB_ERR_ARG, "ib_delta_prepare: %d heads on %d (q, k) heads of %d, values of %d", n_heads, n_qk, d, dv);
    if (filt_w && taps > 1 && !tails) return ib::fail(IB_ERR_ARG, "ib_delta_prepare: a filter of %d taps needs tails", taps);
    if (ldp < 2 * int64_t(n_qk) * d + int64_t(n_heads) * dv + 2 * n_heads + n_qk) return ib::fail(IB_ERR_ARG, "ib_delta_prepare: prepared rows too short");
    const int64_t warps = n_tokens * (n_qk + n_heads + 1);
    IB_LAUNCH(delta_prepare_kernel, blocks_for(warps, 4), 128, 0, rows, ld, col0, a_col, b_col, filt_w, filt_w ? taps : 0, tails,
              (filt_w && taps > 1) ? inline_tail : 0, a_log,
              dt_bias, unit_eps, q_scale, token_seg, seg_start, seg_slot, prep, ldp, n_tokens, n_heads, n_qk, d, dv);
    return ib::check_launch("ib_delta_prepare");
}

IB_EXPORT int ib_tail_update(const float* rows, int64_t ld, int col0, int channels, int taps, float* tails, const int* seg_start,
                             const int* seg_slot, int n_segments, cudaStream_t stream) {
    if (n_segments <= 0 || channels <= 0 || taps <= 1) return IB_OK;
    if (n_segments > 65535) return ib::fail(IB_ERR_ARG, "ib_tail_update: too many segments");
    const dim3 grid{blocks_for(channels, 128), unsigned(n_segments), 1u};
    IB_LAUNCH(tail_update_kernel, grid, 128, 0, rows, ld, col0, channels, taps, tails, seg_start, seg_slot);
    return ib::check_launch("ib_tail_update");
}

// The largest key size a head of ib_state_scan may have.
IB_EXPORT int ib_state_scan_max_dim() { return LK * 32; }

template <int R, int MODE>
static int launch_scan(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* rows, int64_t ld, int q_col,
                       int k_col, int v_col, const float* aux, int64_t lda, int aux_col, float* state, const int* seg_start,
                       const int* seg_slot, float* raw_out, int n_heads, int hpq, int d, int dv, int cb, int chunk, int write_state,
                       int pipelined, const float* bonus, int act) {
    IB_LAUNCH((state_scan_kernel<R, MODE>), grid, threads, smem, rows, ld, q_col, k_col, v_col, aux, lda, aux_col, state, seg_start,
              seg_slot, raw_out, n_heads, hpq, d, dv, cb, chunk, write_state, pipelined, bonus, act);
    return ib::check_launch("ib_state_scan");
}

// mode 0: a decay per key channel (aux: decays at aux_col + h d); mode 1: gated delta rule (aux: g, beta, k.q);
// mode 2: a decay per head (aux: at aux_col + h; lda 0: the same for every token); mode 3: as mode 0 with the read-out
// before the write and `bonus` [heads, d] on the current token.
// `spread` (prompt portions): a head's columns go to more, smaller CTAs until there is about one per SM (sm_count).
IB_EXPORT int ib_state_scan(int mode, const float* rows, int64_t ld, int q_col, int k_col, int v_col, const float* aux,
                            int64_t lda, int aux_col, float* state, const int* seg_start, const int* seg_slot,
                            float* raw_out, int n_segments, int n_heads, int heads_per_qk, int d, int dv, int write_state,
                            int spread, int sm_count, cudaStream_t stream, const float* bonus, int act) {
    if (n_segments <= 0) return IB_OK;
    if (n_heads <= 0 || n_heads > 65535 || heads_per_qk <= 0 || n_heads % heads_per_qk || d <= 0 || dv <= 0 || d > LK * 32)
        return ib::fail(IB_ERR_ARG, "ib_state_scan: %d heads with a state of %d x %d do not fit", n_heads, d, dv);
    if (mode < 0 || mode > 3) return ib::fail(IB_ERR_ARG, "ib_state_scan: unknown mode %d", mode);
    if (mode == 3 && !bonus) return ib::fail(IB_ERR_ARG, "ib_state_scan: mode 3 needs the bonus");
    const bool decay_rows = mode == 0 || mode == 3;
    const int r = d <= 32 ? 4 : (d <= 64 ? 8 : (d <= 128 ? 16 : 32));
    int cb = 32;
    while (cb > 4 && cb / 2 >= dv) cb /= 2;                     // no CTA wider than the head
    if (spread) {
        const int sms = sm_count > 0 ? sm_count : 148;
        while (cb > 8 && n_segments * n_heads * ((dv + cb / 2 - 1) / (cb / 2)) <= sms) cb /= 2;
    }
    // asynchronous copies of rows as they lie need every offset and size on 16 bytes; prompt portions only (a step of
    // single tokens has nothing to copy ahead)
    // act 1: q, k and v are z * sigmoid(z) of what the rows hold, applied while staging (not with copies as they lie)
    const int pipelined = !act && spread && d % 4 == 0 && dv % 4 == 0 && cb % 4 == 0 && ld % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 &&
                          v_col % 4 == 0 && (!decay_rows || (lda % 4 == 0 && aux_col % 4 == 0 && !(uintptr_t(aux) & 15))) &&
                          !(uintptr_t(rows) & 15);
    const int dpp = LK * (r + 4), n_buf = pipelined ? 2 : 1;
    const int per_token = 2 * dpp + (decay_rows ? dpp : 4) + cb;
    int chunk = 11264 / (n_buf * per_token);
    chunk = chunk < 1 ? 1 : (chunk > 16 ? 16 : chunk);
    const size_t smem = size_t(n_buf) * chunk * per_token * sizeof(float);
    if (smem > 48 * 1024) return ib::fail(IB_ERR_ARG, "ib_state_scan: a token of %d floats does not fit the staging area", per_token);
    const dim3 grid{unsigned(n_segments), unsigned(n_heads), unsigned((dv + cb - 1) / cb)};
    const int threads = cb * LK;
#define IB_SCAN(RR, MM)                                                                                                          \
    return launch_scan<RR, MM>(grid, threads, smem, stream, rows, ld, q_col, k_col, v_col, aux, lda, aux_col, state, seg_start, \
                               seg_slot, raw_out, n_heads, heads_per_qk, d, dv, cb, chunk, write_state, pipelined, bonus, act)
    if (mode == 2) {
        if (r == 4) IB_SCAN(4, 2);
        if (r == 8) IB_SCAN(8, 2);
        if (r == 16) IB_SCAN(16, 2);
        IB_SCAN(32, 2);
    }
    if (mode == 3) {
        if (r == 4) IB_SCAN(4, 3);
        if (r == 8) IB_SCAN(8, 3);
        if (r == 16) IB_SCAN(16, 3);
        IB_SCAN(32, 3);
    }
    if (mode == 0) {
        if (r == 4) IB_SCAN(4, 0);
        if (r == 8) IB_SCAN(8, 0);
        if (r == 16) IB_SCAN(16, 0);
        IB_SCAN(32, 0);
    }
    if (r == 4) IB_SCAN(4, 1);
    if (r == 8) IB_SCAN(8, 1);
    if (r == 16) IB_SCAN(16, 1);
    IB_SCAN(32, 1);
#undef IB_SCAN
}

IB_EXPORT int ib_head_norm_gate(const float* o, const float* w, float eps, const void* gate, int64_t ldg, int gate_col,
                                int gate_dtype, void* out, int out_dtype, int64_t n_tokens, int n_heads, int dv,
                                cudaStream_t stream) {
    const int64_t rows = n_tokens * n_heads;
    if (rows <= 0 || dv <= 0) return IB_OK;
    const unsigned grid = blocks_for(rows, 8);
#define IB_HN(TG, TO) IB_LAUNCH((head_norm_gate_kernel<TG, TO>), grid, 256, 0, o, w, eps, (const TG*)gate, ldg, gate_col, (TO*)out, rows, n_heads, dv)
    if (!gate || gate_dtype == IB_F32) {
        if (out_dtype == IB_F32) IB_HN(float, float);
        else if (out_dtype == IB_BF16) IB_HN(float, bf16);
        else return ib::fail(IB_ERR_ARG, "ib_head_norm_gate: unknown dtype %d", out_dtype);
    } else if (gate_dtype == IB_BF16) {
        if (out_dtype == IB_F32) IB_HN(bf16, float);
        else if (out_dtype == IB_BF16) IB_HN(bf16, bf16);
        else return ib::fail(IB_ERR_ARG, "ib_head_norm_gate: unknown dtype %d", out_dtype);
    } else {
        return ib::fail(IB_ERR_ARG, "ib_head_norm_gate: unknown gate dtype %d", gate_dtype);
    }
#undef IB_HN
    return ib::check_launch("ib_head_norm_gate");
}
