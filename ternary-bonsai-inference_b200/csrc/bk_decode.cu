// GQA decode attention over the KV cache: split-K flash decoding, all cache modes.
// Replaces attn_scores*.comp + softmax_inplace.comp + attn_out*.comp (7 dispatches per layer
// in src/gdev.rs:584-829) and the CPU loop src/forward.rs:287-375 with one launch.
//
// Work item = (sequence, kv head, chunk of positions); one CTA of 8 warps per item.  A warp
// takes every 8th position of the chunk; its 32 lanes split the 256 coordinates of a row, so a
// row is read once with full-width coalesced loads and serves all q heads of the GQA group
// (the reference reads every row once per q head).  Scores are completed with xor-shuffle
// reductions, the softmax is the online (running max / running sum) form in the exp2 domain,
// and V is accumulated in registers.  Warps merge through shared memory, CTAs through a
// partials buffer in global memory; the CTA that arrives last for a (sequence, kv head)
// combines the chunks, undoes the Givens rotation for planar V and writes the output, so there
// is no second launch.  No CTA ever waits on another.
//
// Algorithmic traffic per (position, kv head): K row + V row (+ 2 norms); q and out once.
#include <math_constants.h>

#include "bk_decode_common.cuh"

namespace bk {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

// Coordinate held in slot e (0..7) of lane l.  Planar and f16 rows: 8 consecutive coordinates
// (one packed group / one 16-byte load).  f32 rows: two float4 halves 128 coordinates apart so
// that both loads are fully coalesced.
template <int KIND>
__device__ __forceinline__ int dim_of(int lane, int e) {
    if constexpr (KIND == ROW_F32) return (e < 4) ? lane * 4 + e : 128 + lane * 4 + (e - 4);
    else return lane * 8 + e;
}

template <int KIND, int BITS>
struct RawRow {};
template <int BITS>
struct RawRow<ROW_F32, BITS> { float4 a, b; };
template <int BITS>
struct RawRow<ROW_F16, BITS> { uint4 a; };
template <int BITS>
struct RawRow<ROW_PLANAR, BITS> { uint64_t a; float norm; };

template <int KIND, int BITS>
__device__ __forceinline__ RawRow<KIND, BITS> load_row(const uint8_t *rows, const float *norms, size_t r,
                                                       size_t row_bytes, int lane) {
    RawRow<KIND, BITS> x;
    const uint8_t *row = rows + r * row_bytes;
    if constexpr (KIND == ROW_F32) {
        x.a = __ldg(reinterpret_cast<const float4 *>(row) + lane);
        x.b = __ldg(reinterpret_cast<const float4 *>(row) + 32 + lane);
    } else if constexpr (KIND == ROW_F16) {
        x.a = __ldg(reinterpret_cast<const uint4 *>(row) + lane);
    } else {
        x.a = load_group8<BITS>(row, lane);
        x.norm = __ldg(norms + r);
    }
    return x;
}

// Expand a raw row piece to 8 floats (planar: centroid values, norm not applied).
template <int KIND, int BITS>
__device__ __forceinline__ void expand_row(const RawRow<KIND, BITS> &x, const float *sbook, float (&v)[8]) {
    if constexpr (KIND == ROW_F32) {
        v[0] = x.a.x; v[1] = x.a.y; v[2] = x.a.z; v[3] = x.a.w;
        v[4] = x.b.x; v[5] = x.b.y; v[6] = x.b.z; v[7] = x.b.w;
    } else if constexpr (KIND == ROW_F16) {
        const uint32_t w[4] = {x.a.x, x.a.y, x.a.z, x.a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = half_bits_to_f32((uint16_t)(w[i] & 0xffffu));
            v[2 * i + 1] = half_bits_to_f32((uint16_t)(w[i] >> 16));
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = sbook[(uint32_t)(x.a >> (BITS * e)) & ((1u << BITS) - 1u)];
    }
}

template <int KK, int VK, int BITS, int NREP>
__global__ void __launch_bounds__(kThreads) decode_kernel(DecodeArgs a, DecodeMeta meta) {
    __shared__ __align__(16) float s_q[NREP][kHd];       // roped (and rotated) q; later the merged acc
    __shared__ float s_book[256];
    __shared__ float s_m[kWarps][NREP], s_l[kWarps][NREP];
    __shared__ float s_M[NREP], s_L[NREP];
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which item --------------------------------------------------------
    const int item = blockIdx.x;
    int s = 0;
    while (s + 1 < meta.n_seqs && meta.item_start[s + 1] <= item) s++;
    const int n_pos = meta.n_pos[s];
    const int L = meta.chunk_len;
    const int n_chunks = (n_pos + L - 1) / L;
    const int local = item - meta.item_start[s];
    const int kv = local / n_chunks, chunk = local - kv * n_chunks;
    const int p0 = chunk * L, p1 = min(p0 + L, n_pos);
    const int seq = meta.seq_id[s];

    // ---- q: rope, optional Givens rotation, fold scale*log2(e) --------------
    {
        const float *q = a.q + ((size_t)meta.slot[s] * a.n_head + (size_t)kv * NREP) * kHd;
        for (int i = tid; i < NREP * kHd; i += kThreads) (&s_q[0][0])[i] = q[i];
        if (BITS > 0)
            for (int i = tid; i < (1 << BITS); i += kThreads) s_book[i] = a.book[i];
        __syncthreads();
        if (!a.no_rope) {
            const int half = a.n_rot >> 1;
            const float2 *cs = a.rope + (size_t)meta.q_pos[s] * half;
            for (int i = tid; i < NREP * half; i += kThreads) {
                const int r = i / half, j = i - r * half;
                float x0 = s_q[r][j], x1 = s_q[r][j + half];
                rope_pair(x0, x1, cs[j]);
                s_q[r][j] = x0;
                s_q[r][j + half] = x1;
            }
            __syncthreads();
        }
        if (KK == ROW_PLANAR) {
            // K rows hold rotated unit vectors: rotate q once instead (src/forward.rs:304).
            for (int i = tid; i < NREP * (kHd / 2); i += kThreads) {
                const int r = i / (kHd / 2), pr = i - r * (kHd / 2);
                float o0, o1;
                givens_fwd(s_q[r][2 * pr], s_q[r][2 * pr + 1], a.givens[2 * pr], a.givens[2 * pr + 1], o0, o1);
                s_q[r][2 * pr] = o0;
                s_q[r][2 * pr + 1] = o1;
            }
            __syncthreads();
        }
    }
    const float qscale = rsqrtf((float)kHd) * 1.4426950408889634f;  // 1/sqrt(hd) * log2(e)
    float qr[NREP][8];
#pragma unroll
    for (int r = 0; r < NREP; r++)
#pragma unroll
        for (int e = 0; e < 8; e++) qr[r][e] = s_q[r][dim_of<KK>(lane, e)] * qscale;

    // ---- scan --------------------------------------------------------------
    float m[NREP], l[NREP], acc[NREP][8];
#pragma unroll
    for (int r = 0; r < NREP; r++) {
        m[r] = -CUDART_INF_F;
        l[r] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) acc[r][e] = 0.f;
    }
    const size_t seq_rows = (size_t)seq * a.seq_stride_rows;
    int p = p0 + warp;
    RawRow<KK, BITS> kraw{};
    RawRow<VK, BITS> vraw{};
    if (p < p1) {
        const size_t r = seq_rows + (size_t)p * a.n_kv + kv;
        kraw = load_row<KK, BITS>(a.k_rows, a.k_norms, r, a.k_row_bytes, lane);
        vraw = load_row<VK, BITS>(a.v_rows, a.v_norms, r, a.v_row_bytes, lane);
    }
    while (p < p1) {
        const RawRow<KK, BITS> kc = kraw;
        const RawRow<VK, BITS> vc = vraw;
        const int pn = p + kWarps;
        if (pn < p1) {  // prefetch the warp's next position
            const size_t r = seq_rows + (size_t)pn * a.n_kv + kv;
            kraw = load_row<KK, BITS>(a.k_rows, a.k_norms, r, a.k_row_bytes, lane);
            vraw = load_row<VK, BITS>(a.v_rows, a.v_norms, r, a.v_row_bytes, lane);
        }
        float kvv[8];
        expand_row<KK, BITS>(kc, s_book, kvv);
        float sc[NREP];
#pragma unroll
        for (int r = 0; r < NREP; r++) {
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) d = fmaf(qr[r][e], kvv[e], d);
            sc[r] = d;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
#pragma unroll
            for (int r = 0; r < NREP; r++) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], off);
        float vv[8];
        expand_row<VK, BITS>(vc, s_book, vv);
        float vnorm = 1.f;
        if constexpr (VK == ROW_PLANAR) vnorm = vc.norm;
#pragma unroll
        for (int r = 0; r < NREP; r++) {
            float sr = sc[r];
            if constexpr (KK == ROW_PLANAR) sr *= kc.norm;
            if (sr > m[r]) {
                const float corr = exp2f(m[r] - sr);  // 0 on the first position (m = -inf)
                l[r] *= corr;
#pragma unroll
                for (int e = 0; e < 8; e++) acc[r][e] *= corr;
                m[r] = sr;
            }
            const float pr = exp2f(sr - m[r]);
            l[r] += pr;
            const float w = pr * vnorm;
#pragma unroll
            for (int e = 0; e < 8; e++) acc[r][e] = fmaf(w, vv[e], acc[r][e]);
        }
        p = pn;
    }

    // ---- merge the 8 warps --------------------------------------------------
    if (lane == 0)
#pragma unroll
        for (int r = 0; r < NREP; r++) {
            s_m[warp][r] = m[r];
            s_l[warp][r] = l[r];
        }
    __syncthreads();  // also: every warp is done reading s_q
    if (tid < NREP) {
        float M = -CUDART_INF_F;
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, s_m[w][tid]);
        float Lsum = 0.f;
        for (int w = 0; w < kWarps; w++)
            if (s_m[w][tid] > -CUDART_INF_F) Lsum += s_l[w][tid] * exp2f(s_m[w][tid] - M);
        s_M[tid] = M;
        s_L[tid] = Lsum;
    }
    for (int i = tid; i < NREP * kHd; i += kThreads) (&s_q[0][0])[i] = 0.f;
    __syncthreads();
    for (int w = 0; w < kWarps; w++) {  // fixed order keeps the sum deterministic
        if (warp == w) {
#pragma unroll
            for (int r = 0; r < NREP; r++) {
                const float f = (m[r] > -CUDART_INF_F) ? exp2f(m[r] - s_M[r]) : 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) s_q[r][dim_of<VK>(lane, e)] += acc[r][e] * f;
            }
        }
        __syncthreads();
    }

    // ---- merge the chunks of this (sequence, kv head), rotate back, write ------
    const int first_item = meta.item_start[s] + kv * n_chunks;
    finish_item<NREP>(a, meta.slot[s], s, kv, item, n_chunks, first_item, &s_q[0][0], s_M, s_L, &s_last, VK == ROW_PLANAR);
}

// out[row][d] = sum_g acc_g[d] e^{m_g - M} / sum_g l_g e^{m_g - M}
__global__ void lse_merge_kernel(int n_parts, int n_rows, int hd, const float *parts, float *out) {
    const int row = blockIdx.x;
    const int stride = hd + 2;
    float M = -CUDART_INF_F;
    for (int g = 0; g < n_parts; g++) {
        const float *p = parts + ((size_t)g * n_rows + row) * stride;
        if (p[hd + 1] > 0.f) M = fmaxf(M, p[hd]);
    }
    float Ls = 0.f;
    for (int g = 0; g < n_parts; g++) {
        const float *p = parts + ((size_t)g * n_rows + row) * stride;
        if (p[hd + 1] > 0.f) Ls += p[hd + 1] * expf(p[hd] - M);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float sum = 0.f;
        for (int g = 0; g < n_parts; g++) {
            const float *p = parts + ((size_t)g * n_rows + row) * stride;
            if (p[hd + 1] > 0.f) sum = fmaf(p[d], expf(p[hd] - M), sum);
        }
        out[(size_t)row * hd + d] = Ls > 0.f ? sum / Ls : 0.f;
    }
}

template <int KK, int VK, int BITS>
bk_status launch_rep(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m) {
    const int n_rep = a.n_head / a.n_kv;
    switch (n_rep) {
        case 1: decode_kernel<KK, VK, BITS, 1><<<m.n_items, kThreads, 0, ctx->stream>>>(a, m); break;
        case 2: decode_kernel<KK, VK, BITS, 2><<<m.n_items, kThreads, 0, ctx->stream>>>(a, m); break;
        case 4: decode_kernel<KK, VK, BITS, 4><<<m.n_items, kThreads, 0, ctx->stream>>>(a, m); break;
        case 6: decode_kernel<KK, VK, BITS, 6><<<m.n_items, kThreads, 0, ctx->stream>>>(a, m); break;
        case 8: decode_kernel<KK, VK, BITS, 8><<<m.n_items, kThreads, 0, ctx->stream>>>(a, m); break;
        default: return fail(ctx, BK_ERR_UNSUPPORTED, "decode: n_head/n_kv must be 1, 2, 4, 6 or 8");
    }
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace

bk_status launch_decode(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m) {
    if (m.n_items <= 0) return BK_OK;
    if (a.k_kind == ROW_F32 && a.v_kind == ROW_F32) return launch_rep<ROW_F32, ROW_F32, 0>(ctx, a, m);
    if (a.k_kind == ROW_F16 && a.v_kind == ROW_F16) return launch_rep<ROW_F16, ROW_F16, 0>(ctx, a, m);
    if (a.k_kind == ROW_PLANAR) {
        bk_status st = BK_ERR_INVALID;
        const bool vq = a.v_kind == ROW_PLANAR;
        const bool ok = dispatch_bits(a.bits, [&]<int B>() {
            st = vq ? launch_rep<ROW_PLANAR, ROW_PLANAR, B>(ctx, a, m)
                    : launch_rep<ROW_PLANAR, ROW_F32, B>(ctx, a, m);
        });
        if (!ok) return fail(ctx, BK_ERR_INVALID, "decode: bits must be 1..8");
        return st;
    }
    return fail(ctx, BK_ERR_UNSUPPORTED, "decode: unsupported K/V row combination");
}

bk_status launch_lse_merge(bk_ctx *ctx, int n_parts, int n_rows, int hd, const float *parts, float *out) {
    if (n_rows <= 0) return BK_OK;
    lse_merge_kernel<<<n_rows, 256, 0, ctx->stream>>>(n_parts, n_rows, hd, parts, out);
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace bk
