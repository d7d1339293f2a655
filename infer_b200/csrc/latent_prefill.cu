// Attention through low-rank latents for prompt portions, with per-head keys and values formed for the step.
//
// A cached position is one row [c | r] for all heads (latent_ops.cu). A decoded token reads those rows as they are,
// in the latent space. A prompt portion of n tokens would pay kv_rank + rot_dim multiply-adds per (query, key, head)
// that way; forming k_h = W_uk_h c and v_h = W_uv_h c once per visible position (one matrix product over the rows
// that the portions' segments can see) brings that down to head_dim + rot_dim and v_head_dim, and puts both products
// of the attention on the tensor cores. Three steps:
//
//   latent_gather     the rows that the step's portions can see, copied out of the pages into one region per portion
//                     (`span` rows each; row j of a region is position lo + j, lo = the first position any token of the
//                     portion sees); rows past the portion's last token are zero
//   (a matrix product of the gathered c rows with [W_uk; W_uv], by the caller)
//   latent_prefill    per (64 queries of a portion, head): S = Q K^T on mma.sync m16n8k16 (bfloat16 in, float out),
//                     K = [k_h | r], Q's rotated part turned as it is loaded; mask; running softmax in float; the
//                     probabilities enter P V as TWO bfloat16 terms (p = hi + lo, |lo| <= 2^-9 hi), so that the
//                     weights keep 16 bits of mantissa; the result is divided, multiplied by the head's gate and a
//                     constant, and stored
//
// Compiled for one pair of padded sizes: -DIB_QK_DIM (head_dim + rot_dim rounded up to 16) and -DIB_V_DIM (v_head_dim
// rounded up to 16); head_dim, rot_dim and v_head_dim themselves are arguments and multiples of 8.
// Which rows are portions is read from seg_start on the device (segments longer than one token, in order), so a
// captured step can be replayed with other positions; launch sizes depend on the segment lengths and `span` alone.
#include "common.cuh"

IB_DEFINE_LAST_ERROR()

#ifndef IB_QK_DIM
#define IB_QK_DIM 192
#endif
#ifndef IB_V_DIM
#define IB_V_DIM 128
#endif

#define IB_LAUNCH(kernel, grid, block, smem, ...)                                                              \
    do {                                                                                                       \
        const int rc_ = ib::launch(#kernel, kernel, dim3(grid), dim3(block), size_t(smem), stream, 1u, __VA_ARGS__); \
        if (rc_) return rc_;                                                                                   \
    } while (0)

namespace {

using bf16 = __nv_bfloat16;
constexpr int DQK = IB_QK_DIM, DV = IB_V_DIM;
static_assert(DQK % 16 == 0 && DV % 16 == 0 && DQK >= 16 && DV >= 16 && DQK <= 512 && DV <= 128, "padded sizes");
constexpr int BM = 64, BN = 64, PF_THREADS = 128;
constexpr int QS = DQK + 8, VS = DV + 8;                     // shared-memory row strides in elements: an odd number of 16-byte units
constexpr float LOG2E = 1.4426950408889634f;

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
// 16 bytes from global to shared memory without passing registers; `bytes` 0: sixteen zero bytes, nothing is read
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// p = hi + lo in bfloat16: hi the rounding of p, lo the rounding of what is left
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack2(x - hf.x, y - hf.y);
}

// The p-th segment longer than one token: its index, or -1.
__device__ __forceinline__ int portion_segment(const int* __restrict__ seg_start, int n_seg, int p) {
    int seen = 0;
    for (int s = 0; s < n_seg; s++) {
        if (seg_start[s + 1] - seg_start[s] > 1) {
            if (seen == p) return s;
            seen++;
        }
    }
    return -1;
}

// ------------------------------------------------------------------------------------------------
// One warp per gathered row. c_out [P * span][kv_rank], r_out [P * span][dr]; 16-byte copies (kv_rank, dr and
// kv_rank + dr are multiples of 8 elements).
constexpr int GA_WARPS = 8;

__global__ void __launch_bounds__(GA_WARPS * 32)
latent_gather_kernel(const bf16* __restrict__ cache, const int* __restrict__ block_table, int64_t max_blocks,
                     const int* __restrict__ seg_start, const int* __restrict__ seg_pos0, int n_seg, int span, int window,
                     int page_size, int64_t n_pages, int kv_rank, int dr, bf16* __restrict__ c_out, bf16* __restrict__ r_out,
                     int64_t n_rows, int* status) {
    ib::pdl_wait();
    const int64_t row = int64_t(blockIdx.x) * GA_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int p = int(row / span), j = int(row - int64_t(p) * span);
    const int s = portion_segment(seg_start, n_seg, p);
    const bf16* src = nullptr;
    if (s >= 0) {
        const int pos0 = seg_pos0[s], last = pos0 + (seg_start[s + 1] - seg_start[s]) - 1;
        const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
        const int pos = lo + j;
        if (pos <= last) {
            const int page = block_table[int64_t(s) * max_blocks + pos / page_size];
            if (page < 0 || page >= n_pages) {
                if (status && lane == 0) atomicExch(status, 3);
            } else {
                src = cache + (int64_t(page) * page_size + pos % page_size) * (kv_rank + dr);
            }
        }
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4* cd = reinterpret_cast<uint4*>(c_out + row * kv_rank);
    uint4* rd = reinterpret_cast<uint4*>(r_out + row * dr);
    const uint4* sv = reinterpret_cast<const uint4*>(src);
    const int nc = kv_rank / 8, nr = dr / 8;
    for (int i = lane; i < nc; i += 32) cd[i] = src ? sv[i] : zero;
    for (int i = lane; i < nr; i += 32) rd[i] = src ? sv[nc + i] : zero;
}

// ------------------------------------------------------------------------------------------------
// q [T][H * (d + dr)] as the query up-projection leaves it (a head's unrotated channels, then its rotated ones, not
// yet turned); kv [P * span][ld_kv]: a gathered row's per-head keys at column h * d, its per-head values at column
// v_col + h * dv; r [P * span][dr] the gathered shared key parts (already turned); out [T][H * dv].
__global__ void __launch_bounds__(PF_THREADS)
latent_prefill_kernel(const bf16* __restrict__ q, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int layout,
                      int n_rot, const bf16* __restrict__ kv, int64_t ld_kv, int v_col, const bf16* __restrict__ r,
                      const float* __restrict__ gates, int64_t gate_ld, int gate_col, float mult, bf16* __restrict__ out,
                      const int* __restrict__ seg_start, const int* __restrict__ seg_pos0, int n_seg, int span, int n_heads,
                      int d, int dr, int dv, int window, float scale) {
    ib::pdl_wait();
    extern __shared__ __align__(16) unsigned char pf_sm[];
    bf16* Qs = reinterpret_cast<bf16*>(pf_sm);               // [BM][QS]
    bf16* Ks = Qs + BM * QS;                                 // [BN][QS]
    bf16* Vs = Ks + BN * QS;                                 // [BN][VS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, h = blockIdx.y;
    // which portion and which of its query tiles
    int tile = blockIdx.x, p = 0, s = -1, len = 0;
    for (int i = 0; i < n_seg; i++) {
        const int n = seg_start[i + 1] - seg_start[i];
        if (n <= 1) continue;
        const int nt = (n + BM - 1) / BM;
        if (tile < nt) { s = i; len = n; break; }
        tile -= nt;
        p++;
    }
    if (s < 0) return;
    tile = (len + BM - 1) / BM - 1 - tile;                   // a portion's last queries see the most keys: they start first
    const int q0 = tile * BM, t0 = seg_start[s] + q0, pos0 = seg_pos0[s];
    const int nq = min(BM, len - q0);
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int qp_first = pos0 + q0, qp_last = qp_first + nq - 1;
    const int k_min = window > 0 ? max(0, qp_first - window + 1) : 0;
    const int j_first = k_min - lo, j_last = min(qp_last - lo, span - 1);
    const int dh = d + dr, ldq = n_heads * dh;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    // Q: the unrotated channels as they are, the rotated ones turned by the token's position, the padding zero
    {
        const int cpr = d / 8;
        for (int i = tid; i < BM * cpr; i += PF_THREADS) {
            const int row = i / cpr, e = (i - row * cpr) * 8;
            *reinterpret_cast<uint4*>(Qs + row * QS + e) =
                row < nq ? *reinterpret_cast<const uint4*>(q + int64_t(t0 + row) * ldq + h * dh + e) : zero4;
        }
        const int tail = DQK - d, half = n_rot / 2;
        for (int i = tid; i < BM * tail; i += PF_THREADS) {
            const int row = i / tail, e = i - row * tail;
            float val = 0.0f;
            if (row < nq && e < dr) {
                const bf16* src = q + int64_t(t0 + row) * ldq + h * dh + d;
                if (e < n_rot) {
                    const int j = layout == 0 ? e >> 1 : (e < half ? e : e - half);
                    const int a = layout == 0 ? 2 * j : j, b = layout == 0 ? 2 * j + 1 : j + half;
                    const int64_t ti = int64_t(pos0 + q0 + row) * half + j;
                    const float c = cos_t[ti], sn = sin_t[ti];
                    const float u = __bfloat162float(src[a]), v = __bfloat162float(src[b]);
                    val = e == a ? u * c - v * sn : v * c + u * sn;
                } else {
                    val = __bfloat162float(src[e]);
                }
            }
            Qs[row * QS + d + e] = __float2bfloat16_rn(val);
        }
    }

    const int ra = warp * 16 + (lane >> 2), rb = ra + 8;     // this thread's two query rows of the tile
    const int qpa = ra < nq ? qp_first + ra : -1, qpb = rb < nq ? qp_first + rb : -1;
    const int wq_min = qp_first + warp * 16, wq_max = min(wq_min + 15, qp_last);   // the warp's query positions
    const bool warp_full = warp * 16 + 15 < nq;
    const float sl2 = scale * LOG2E;                         // scores are kept times log2(e): exponentials are exp2
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    // K and V tiles have one buffer each and are asked for one tile ahead: K(j + 1) as soon as S(j) has been
    // computed, V(j + 1) as soon as P(j) V(j) has; each request is one cp.async group.
    const int64_t region = int64_t(p) * span;
    auto load_k = [&](int j0) {
        constexpr int cpr = DQK / 8;
        for (int i = tid; i < BN * cpr; i += PF_THREADS) {
            const int row = i / cpr, e = (i - row * cpr) * 8, j = j0 + row;
            const bf16* src = kv;
            int bytes = 0;
            if (j < span) {
                const int64_t g = region + j;
                if (e < d) { src = kv + g * ld_kv + h * d + e; bytes = 16; }
                else if (e < dh) { src = r + g * dr + (e - d); bytes = 16; }
            }
            cp_async16(smem_u32(Ks + row * QS + e), src, bytes);
        }
        cp_async_commit();
    };
    auto load_v = [&](int j0) {
        constexpr int vpr = DV / 8;
        for (int i = tid; i < BN * vpr; i += PF_THREADS) {
            const int row = i / vpr, e = (i - row * vpr) * 8, j = j0 + row;
            const bf16* src = kv;
            int bytes = 0;
            if (j < span && e < dv) { src = kv + (region + j) * ld_kv + v_col + h * dv + e; bytes = 16; }
            cp_async16(smem_u32(Vs + row * VS + e), src, bytes);
        }
        cp_async_commit();
    };
    const int jt_first = j_first / BN, jt_last = j_last / BN;
    load_k(jt_first * BN);
    load_v(jt_first * BN);
    for (int jt = jt_first; jt <= jt_last; jt++) {
        const int j0 = jt * BN;
        const int kp_lo = lo + j0, kp_hi = kp_lo + BN - 1;
        // the warp's part of this tile: nothing visible, everything visible, or masked element by element
        const bool none = kp_lo > wq_max || (window > 0 && wq_min - kp_hi >= window);
        const bool all = warp_full && kp_hi <= wq_min && (window <= 0 || wq_max - kp_lo < window) && j0 + BN <= span;
        cp_async_wait<1>();                                  // K(j) has arrived (V(j) may still be on its way)
        __syncthreads();
        float sc[BN / 8][4];
        if (!none) {
#pragma unroll
            for (int i = 0; i < BN / 8; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
#pragma unroll 2
            for (int ks = 0; ks < DQK / 16; ks++) {
                uint32_t a[4];
                ldsm4(smem_u32(Qs + (warp * 16 + (lane & 15)) * QS + ks * 16 + (lane >> 4) * 8), a);
#pragma unroll
                for (int np = 0; np < BN / 16; np++) {
                    uint32_t b[4];
                    ldsm4(smem_u32(Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * QS + ks * 16 + ((lane >> 3) & 1) * 8), b);
                    mma16816(sc[2 * np], a, b[0], b[1]);
                    mma16816(sc[2 * np + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                     // every warp has read K(j)
        if (jt < jt_last) load_k(j0 + BN); else cp_async_commit();
        float al_a = 1.0f, al_b = 1.0f;
        if (!none) {
            float mx_a = -INFINITY, mx_b = -INFINITY;
            if (all) {
#pragma unroll
                for (int nt = 0; nt < BN / 8; nt++) {
#pragma unroll
                    for (int c = 0; c < 4; c++) sc[nt][c] *= sl2;
                    mx_a = fmaxf(mx_a, fmaxf(sc[nt][0], sc[nt][1]));
                    mx_b = fmaxf(mx_b, fmaxf(sc[nt][2], sc[nt][3]));
                }
            } else {
                const int kp0 = kp_lo + (lane & 3) * 2;
#pragma unroll
                for (int nt = 0; nt < BN / 8; nt++) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const int kp = kp0 + nt * 8 + (c & 1), qp = c < 2 ? qpa : qpb;
                        const bool vis = kp <= qp && (window <= 0 || qp - kp < window) && kp - lo < span;
                        const float v = vis ? sc[nt][c] * sl2 : -INFINITY;
                        sc[nt][c] = v;
                        if (c < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                    }
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            al_a = m_a == -INFINITY ? 0.0f : exp2f(m_a - mn_a);
            al_b = m_b == -INFINITY ? 0.0f : exp2f(m_b - mn_b);
            const float ba = mn_a == -INFINITY ? 0.0f : mn_a, bb = mn_b == -INFINITY ? 0.0f : mn_b;
            m_a = mn_a;
            m_b = mn_b;
            float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
            for (int nt = 0; nt < BN / 8; nt++) {
                sc[nt][0] = exp2f(sc[nt][0] - ba);           // exp2(-inf) = 0 for what is masked
                sc[nt][1] = exp2f(sc[nt][1] - ba);
                sc[nt][2] = exp2f(sc[nt][2] - bb);
                sc[nt][3] = exp2f(sc[nt][3] - bb);
                sum_a += sc[nt][0] + sc[nt][1];
                sum_b += sc[nt][2] + sc[nt][3];
            }
            l_a = l_a * al_a + sum_a;
            l_b = l_b * al_b + sum_b;
#pragma unroll
            for (int i = 0; i < DV / 8; i++) {
                o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b;
            }
        }
        cp_async_wait<1>();                                  // V(j) has arrived (K(j + 1) may still be on its way)
        __syncthreads();
        if (!none) {
            // O += P V, P as two bfloat16 terms
#pragma unroll
            for (int kk = 0; kk < BN / 16; kk++) {
                uint32_t ph[4], pl[4];
                split2(sc[2 * kk][0], sc[2 * kk][1], ph[0], pl[0]);
                split2(sc[2 * kk][2], sc[2 * kk][3], ph[1], pl[1]);
                split2(sc[2 * kk + 1][0], sc[2 * kk + 1][1], ph[2], pl[2]);
                split2(sc[2 * kk + 1][2], sc[2 * kk + 1][3], ph[3], pl[3]);
                // two channel tiles at a time: four products lie between the two that add into one accumulator
#pragma unroll
                for (int np = 0; np + 1 < DV / 16; np += 2) {
                    uint32_t b[4], c[4];
                    const uint32_t at = smem_u32(Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + np * 16 + (lane >> 4) * 8);
                    ldsm4_t(at, b);
                    ldsm4_t(at + 32, c);
                    mma16816(o[2 * np], ph, b[0], b[1]);
                    mma16816(o[2 * np + 1], ph, b[2], b[3]);
                    mma16816(o[2 * np + 2], ph, c[0], c[1]);
                    mma16816(o[2 * np + 3], ph, c[2], c[3]);
                    mma16816(o[2 * np], pl, b[0], b[1]);
                    mma16816(o[2 * np + 1], pl, b[2], b[3]);
                    mma16816(o[2 * np + 2], pl, c[0], c[1]);
                    mma16816(o[2 * np + 3], pl, c[2], c[3]);
                }
                if ((DV / 16) % 2) {
                    constexpr int np = DV / 16 - 1;
                    uint32_t b[4];
                    ldsm4_t(smem_u32(Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + np * 16 + (lane >> 4) * 8), b);
                    mma16816(o[2 * np], ph, b[0], b[1]);
                    mma16816(o[2 * np + 1], ph, b[2], b[3]);
                    mma16816(o[2 * np], pl, b[0], b[1]);
                    mma16816(o[2 * np + 1], pl, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                     // every warp has read V(j)
        if (jt < jt_last) load_v(j0 + BN); else cp_async_commit();
    }
    cp_async_wait<0>();
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
#pragma unroll
    for (int half_i = 0; half_i < 2; half_i++) {
        const int row = half_i ? rb : ra;
        if (row >= nq) continue;
        const int64_t t = t0 + row;
        const float l = half_i ? l_b : l_a;
        float f = (l > 0.0f ? 1.0f / l : 0.0f) * mult;
        if (gates) f *= 1.0f / (1.0f + expf(-gates[t * gate_ld + gate_col + h]));
        bf16* dst = out + (t * n_heads + h) * dv;
#pragma unroll
        for (int i = 0; i < DV / 8; i++) {
            const int col = i * 8 + (lane & 3) * 2;
            if (col < dv)
                *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[i][2 * half_i] * f, o[i][2 * half_i + 1] * f);
        }
    }
}

}  // namespace

IB_EXPORT int ib_latent_prefill_dims(int* qk, int* v) {
    *qk = DQK;
    *v = DV;
    return IB_OK;
}

// n_rows = portions * span. The rows of every portion are written (zeros past its last token).
IB_EXPORT int ib_latent_gather(const void* cache, const int* block_table, int64_t max_blocks, const int* seg_start, const int* seg_pos0,
                               int n_seg, int span, int window, int page_size, int64_t n_pages, int kv_rank, int dr, void* c_out,
                               void* r_out, int64_t n_rows, int* status, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (kv_rank <= 0 || kv_rank % 8 || dr <= 0 || dr % 8 || span <= 0 || n_seg <= 0 || page_size <= 0)
        return ib::fail(IB_ERR_ARG, "ib_latent_gather: rows of %d + %d in regions of %d", kv_rank, dr, span);
    IB_LAUNCH(latent_gather_kernel, unsigned((n_rows + GA_WARPS - 1) / GA_WARPS), GA_WARPS * 32, 0, (const bf16*)cache, block_table, max_blocks,
              seg_start, seg_pos0, n_seg, span, window, page_size, n_pages, kv_rank, dr, (bf16*)c_out, (bf16*)r_out, n_rows, status);
    return ib::check_launch("ib_latent_gather");
}

// n_tiles: the sum over the step's portions of ceil(length / 64).
IB_EXPORT int ib_latent_prefill(const void* q, const float* cos_t, const float* sin_t, int layout, int n_rot, const void* kv, int64_t ld_kv,
                                int v_col, const void* r, const float* gates, int64_t gate_ld, int gate_col, float mult, void* out,
                                const int* seg_start, const int* seg_pos0, int n_seg, int span, int n_tiles, int n_heads, int d, int dr,
                                int dv, int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return IB_OK;
    if (d <= 0 || d % 8 || dr <= 0 || dr % 8 || dv <= 0 || dv % 8 || d + dr > DQK || dv > DV || ld_kv % 8 || v_col % 8)
        return ib::fail(IB_ERR_ARG, "ib_latent_prefill: heads of %d + %d and %d do not fit this build (%d, %d)", d, dr, dv, DQK, DV);
    if (n_rot < 0 || n_rot % 2 || n_rot > dr || (n_rot && (!cos_t || !sin_t)) || n_heads <= 0 || n_heads > 65535 || span <= 0)
        return ib::fail(IB_ERR_ARG, "ib_latent_prefill: %d rotated channels of %d, %d heads, regions of %d", n_rot, dr, n_heads, span);
    const size_t smem = size_t(BM + BN) * QS * sizeof(bf16) + size_t(BN) * VS * sizeof(bf16);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(latent_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return ib::fail(IB_ERR_CUDA, "ib_latent_prefill: shared memory of %zu bytes: %s", smem, cudaGetErrorString(e));
    }
    IB_LAUNCH(latent_prefill_kernel, dim3(unsigned(n_tiles), unsigned(n_heads)), PF_THREADS, smem, (const bf16*)q, cos_t, sin_t, layout, n_rot,
              (const bf16*)kv, ld_kv, v_col, (const bf16*)r, gates, gate_ld, gate_col, mult, (bf16*)out, seg_start, seg_pos0, n_seg, span,
              n_heads, d, dr, dv, window, scale);
    return ib::check_launch("ib_latent_prefill");
}
