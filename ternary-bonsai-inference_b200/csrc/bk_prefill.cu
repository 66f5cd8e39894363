// Causal attention of a block of prompt tokens over a 4-bit or 3-bit planar cache: the batched
// (prefill) form of the decode attention.  The reference refuses a batched pass over a quantized
// cache (src/gdev.rs:1366-1372) and runs the prompt token by token through the decode path
// (src/forward.rs:247-375 per token); this kernel gives the same result per token and reads
// every cache row once per block of query rows instead of once per token.
//
// Work item = (query block, kv head, context chunk); one CTA of 8 warps.  A query block is up
// to 128 query rows = consecutive (token, q head of the GQA group) pairs, 16 rows per warp.
// Per tile of 32 positions the CTA dequantizes the packed K and V rows ONCE into shared memory
// as f16 hi + lo tiles (alpha-scaled centroids and their rounding remainders: a token early in
// the prompt sees few rows, so nothing averages the 1e-4 of a single f16 table out; rows of 512
// bytes in four 128-byte slabs with the chunk ^ (row & 7) swizzle, so every ldmatrix is conflict-free),
// and every warp then contracts its 16 query rows against the tile on the tensor cores
// (mma.sync.m16n8k16, f16 in, f32 accumulate):
//     S[16 rows x 32 pos]  = Q[16 x 256] . K^T      (A = q from shared memory; q_hi k_hi + q_lo k_hi + q_hi k_lo)
//     O[16 rows x 256]    += W[16 x 32] . V         (A = softmax weights straight from the S registers, f16 hi + lo)
// The norms stay outside the f16 operands: scores are scaled by ||k|| per column, and the
// weights carry p * ||v|| referenced to the running maximum of s + log2 ||v|| (times 2^14), as in
// the decode kernel.  Online softmax per query row; causal limit per row (token i sees positions
// 0 .. pos0 + i).  The packed rows of the next tile are fetched into registers while the current
// one is computed.  With more than one context chunk the CTAs write (O, m, l) triples and a second
// small kernel merges them; the inverse Givens rotation of the output is applied where the
// final row is written.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <atomic>

#include "bk_device.cuh"
#include "bk_internal.h"
#include "bk_mma_common.cuh"

namespace bk {

namespace {

constexpr int kPW = 8;            // warps per CTA
constexpr int kPT = kPW * 32;
constexpr int kQRows = 16 * kPW;  // query rows per CTA
constexpr int kTK = 32;           // positions per tile
constexpr float kWScale = 16384.0f;

constexpr uint32_t kQTileBytes = 4 * kQRows * 128;  // 64 KiB: [4 slabs][128 rows][128 B]
constexpr uint32_t kKVTileBytes = 4 * kTK * 128;    // 16 KiB: [4 slabs][32 rows][128 B]
struct Small {
    float kn[kTK], vn[kTK];
    float givens[kHd];
    __half table[16], table_lo[16];  // alpha * c rounded to f16, and what the rounding left
};
constexpr uint32_t kPrefillSmem = 2 * kQTileBytes + 4 * kKVTileBytes + sizeof(Small);

// byte offset of 16-byte chunk `chunk` (0..31: 8 coordinates each) of row `row` in a tile of `rows` rows
__device__ __forceinline__ uint32_t tile_off(int rows, int row, int chunk) {
    return (uint32_t)((chunk >> 3) * rows * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t expand24p(uint32_t y) {
    y &= 0x00ffffffu;
    y += (y & 0x00fff000u) * 15u;
    y += (y & 0x0fc00fc0u) * 3u;
    y += (y & 0x38383838u);
    return y;
}

struct PrefillArgs {
    DecodeArgs d;        // cache pointers, tables, q, out (q/out: [n_tokens][n_head][hd])
    int seq, pos0, n_tokens;
    int tq;              // tokens per query block
    int n_blocks, n_chunks;
    float lut_alpha;
    float *scratch;      // [n_tokens * n_head][n_chunks][kHd + 2] when n_chunks > 1
};

// 32 coordinates (four words of eight nibbles) -> 32 halfs, stored as four 16-byte chunks
__device__ __forceinline__ void dequant_store(const uint32_t (&w)[4], const __half *table, uint8_t *tile, int row, int chunk0) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t h[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const uint32_t lo = (w[j] >> (8 * e)) & 15u, hi = (w[j] >> (8 * e + 4)) & 15u;
            h[e] = (uint32_t)__half_as_ushort(table[lo]) | ((uint32_t)__half_as_ushort(table[hi]) << 16);
        }
        *reinterpret_cast<uint4 *>(tile + tile_off(kTK, row, chunk0 + j)) = make_uint4(h[0], h[1], h[2], h[3]);
    }
}

template <int BITS, int NREP>
__global__ void __launch_bounds__(kPT, 1) prefill_mma_kernel(PrefillArgs pa) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const DecodeArgs &a = pa.d;
    uint8_t *q_hi = smem, *q_lo = smem + kQTileBytes;
    uint8_t *k_tile = smem + 2 * kQTileBytes, *v_tile = k_tile + kKVTileBytes, *vl_tile = v_tile + kKVTileBytes;
    uint8_t *kl_tile = vl_tile + kKVTileBytes;
    Small &sm = *reinterpret_cast<Small *>(kl_tile + kKVTileBytes);
    const uint32_t q_hi_s = (uint32_t)__cvta_generic_to_shared(q_hi), q_lo_s = q_hi_s + kQTileBytes;
    const uint32_t k_s = q_hi_s + 2 * kQTileBytes, v_s = k_s + kKVTileBytes, vl_s = v_s + kKVTileBytes, kl_s = vl_s + kKVTileBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    constexpr int kRowBytes = 32 * BITS;
    // The eight 3-bit centroids round to f16 within 2e-5 under the context's alpha, the sixteen
    // 4-bit ones only within 1e-4: the 4-bit kernel carries the rounding remainders as lo tiles.
    constexpr bool kLoTiles = BITS == 4;

    // ---- which item ------------------------------------------------------------------------
    const int item = blockIdx.x;
    // the blocks late in the prompt see the most rows: they go first
    const int chunk = item % pa.n_chunks, kv = (item / pa.n_chunks) % a.n_kv, blk = pa.n_blocks - 1 - item / (pa.n_chunks * a.n_kv);
    const int tok0 = blk * pa.tq, n_tok = min(pa.tq, pa.n_tokens - tok0), n_rows = n_tok * NREP;
    const int vis = pa.pos0 + tok0 + n_tok;  // positions the last token of the block sees
    const int L = ((vis + pa.n_chunks - 1) / pa.n_chunks + kTK - 1) / kTK * kTK;
    const int c0 = chunk * L, c1 = min(c0 + L, vis);
    const int n_tiles = c1 > c0 ? (c1 - c0 + kTK - 1) / kTK : 0;

    // ---- tables ------------------------------------------------------------------------------
    for (int i = tid; i < kHd; i += kPT) sm.givens[i] = a.givens[i];
    if (tid < 16) {
        const float c = a.book[tid & ((1 << BITS) - 1)] * pa.lut_alpha;
        const __half h = __float2half_rn(c);
        sm.table[tid] = h;
        sm.table_lo[tid] = __float2half_rn(c - __half2float(h));
    }
    __syncthreads();

    // ---- q rows: rope at the token's position, Givens rotation, scale, f16 hi/lo into the two
    // q tiles (a warp per row, staged through the K tile area) ---------------------------------
    {
        float *stage = reinterpret_cast<float *>(k_tile) + warp * (kHd + 8);  // rows are padded by one float per 32 (see pad())
        auto pad = [](int i) { return i + (i >> 5); };  // lanes 8 coordinates apart land in different banks
        const float qscale = rsqrtf((float)kHd) * 1.4426950408889634f / pa.lut_alpha;
        const int half = a.n_rot >> 1;
        // the next row's q and rope values travel while the current row is processed
        float xn[8];
        float2 rn[4];
        auto prefetch = [&](int r) {
            if (r < n_rows) {
                const int tok = tok0 + r / NREP, head = kv * NREP + r % NREP;
                const float *src = a.q + ((size_t)tok * a.n_head + head) * kHd;
                const float2 *cs = a.rope + (size_t)(pa.pos0 + tok) * half;
#pragma unroll
                for (int i = 0; i < 8; i++) xn[i] = __ldg(src + lane + 32 * i);
#pragma unroll
                for (int i = 0; i < 4; i++) rn[i] = (lane + 32 * i < half) ? __ldg(cs + lane + 32 * i) : make_float2(1.f, 0.f);
            }
        };
        prefetch(warp);
        for (int r = warp; r < kQRows; r += kPW) {
            const bool real = r < n_rows;
            if (real) {
                float2 rc[4];
#pragma unroll
                for (int i = 0; i < 8; i++) stage[pad(lane + 32 * i)] = xn[i];
#pragma unroll
                for (int i = 0; i < 4; i++) rc[i] = rn[i];
                prefetch(r + kPW);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int j = lane + 32 * i;
                    if (j < half) {
                        float x0 = stage[pad(j)], x1 = stage[pad(j + half)];
                        rope_pair(x0, x1, rc[i]);
                        stage[pad(j)] = x0;
                        stage[pad(j + half)] = x1;
                    }
                }
                __syncwarp();
            }
            // lane handles coordinates 8 lane .. 8 lane + 7 = one 16-byte chunk of each tile
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                float o0 = 0.f, o1 = 0.f;
                if (real) {
                    const int d = 8 * lane + 2 * p;
                    givens_fwd(stage[pad(d)], stage[pad(d + 1)], sm.givens[d], sm.givens[d + 1], o0, o1);
                    o0 *= qscale;
                    o1 *= qscale;
                }
                const __half h0 = __float2half_rn(o0), h1 = __float2half_rn(o1);
                const __half l0 = __float2half_rn(o0 - __half2float(h0)), l1 = __float2half_rn(o1 - __half2float(h1));
                hw[p] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
                lw[p] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
            }
            const uint32_t off = tile_off(kQRows, r, lane);
            *reinterpret_cast<uint4 *>(q_hi + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4 *>(q_lo + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            __syncwarp();
        }
    }

    // ---- per-thread share of a packed tile: position tid / 8, coordinates 32 (tid % 8) .. + 31 ----
    const int my_row = tid >> 3, my_c = tid & 7;
    const size_t seq_rows = (size_t)pa.seq * a.seq_stride_rows;
    uint32_t pk[4], pv[4];
    float pn = 0.f;
    auto fetch = [&](int tile) {
        const int pos = min(c0 + tile * kTK + my_row, a.n_ctx - 1);  // rows past the chunk are masked, never out of the cache
        const size_t row = seq_rows + (size_t)pos * a.n_kv + kv;
        const uint8_t *kr = a.k_rows + row * kRowBytes, *vr = a.v_rows + row * kRowBytes;
        if constexpr (BITS == 4) {
            const uint4 x = __ldg(reinterpret_cast<const uint4 *>(kr) + my_c), y = __ldg(reinterpret_cast<const uint4 *>(vr) + my_c);
            pk[0] = x.x; pk[1] = x.y; pk[2] = x.z; pk[3] = x.w;
            pv[0] = y.x; pv[1] = y.y; pv[2] = y.z; pv[3] = y.w;
        } else {  // 12 bytes = 32 indices of 3 bits
            const uint32_t *k3 = reinterpret_cast<const uint32_t *>(kr) + 3 * my_c, *v3 = reinterpret_cast<const uint32_t *>(vr) + 3 * my_c;
            pk[0] = __ldg(k3); pk[1] = __ldg(k3 + 1); pk[2] = __ldg(k3 + 2); pk[3] = 0;
            pv[0] = __ldg(v3); pv[1] = __ldg(v3 + 1); pv[2] = __ldg(v3 + 2); pv[3] = 0;
        }
        // norms of the tile: threads 0..31 fetch K's, 32..63 V's
        if (tid < 2 * kTK) {
            const int p2 = min(c0 + tile * kTK + (tid & (kTK - 1)), a.n_ctx - 1);
            const size_t r2 = seq_rows + (size_t)p2 * a.n_kv + kv;
            pn = __ldg((tid < kTK ? a.k_norms : a.v_norms) + r2);
        }
    };
    auto widen = [&](uint32_t (&w)[4]) {
        if constexpr (BITS == 3) {
            const uint32_t u0 = w[0], u1 = w[1], u2 = w[2];
            w[0] = expand24p(u0);
            w[1] = expand24p(__funnelshift_r(u0, u1, 24));
            w[2] = expand24p(__funnelshift_r(u1, u2, 16));
            w[3] = expand24p(u2 >> 8);
        }
    };

    float acc[32][4];
#pragma unroll
    for (int j = 0; j < 32; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    float M0 = -CUDART_INF_F, M1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    // causal limits of this lane's two rows (positions < lim are visible); rows past the block see nothing
    const int row0 = 16 * warp + g, row1 = row0 + 8;
    const int lim0 = row0 < n_rows ? pa.pos0 + tok0 + row0 / NREP + 1 : 0;
    const int lim1 = row1 < n_rows ? pa.pos0 + tok0 + row1 / NREP + 1 : 0;

    // ldmatrix lane addresses.  A (q rows, plain): matrices (rows 0-7, c), (rows 8-15, c), (rows 0-7, c+1),
    // (rows 8-15, c+1).  B from K (plain): (pos 0-7, c), (pos 0-7, c+1), (pos 8-15, c), (pos 8-15, c+1).
    // B from V (transposed): (pos 0-7, c), (pos 8-15, c), (pos 0-7, c+1), (pos 8-15, c+1).
    const int a_row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8, a_c = lane >> 4;
    const int bk_row = (lane & 7) + (lane >> 4) * 8, bk_c = (lane >> 3) & 1;
    const int bv_row = (lane & 7) + ((lane >> 3) & 1) * 8, bv_c = lane >> 4;

    // positions below warp_lim are visible to at least one row of this warp
    const int last_row = min(16 * warp + 15, n_rows - 1);
    const int warp_lim = last_row >= 16 * warp ? pa.pos0 + tok0 + last_row / NREP + 1 : 0;

    if (n_tiles > 0) fetch(0);
    for (int tile = 0; tile < n_tiles; tile++) {
        __syncthreads();  // the previous tile has been consumed (first pass: the q staging is over)
        widen(pk);
        widen(pv);
        dequant_store(pk, sm.table, k_tile, my_row, 4 * my_c);
        if constexpr (kLoTiles) dequant_store(pk, sm.table_lo, kl_tile, my_row, 4 * my_c);
        dequant_store(pv, sm.table, v_tile, my_row, 4 * my_c);
        if constexpr (kLoTiles) dequant_store(pv, sm.table_lo, vl_tile, my_row, 4 * my_c);
        if (tid < kTK) sm.kn[tid] = pn;
        else if (tid < 2 * kTK) sm.vn[tid - kTK] = pn;
        if (tile + 1 < n_tiles) fetch(tile + 1);
        __syncthreads();

        const int pb = c0 + tile * kTK;
        if (pb >= warp_lim) continue;  // nothing of this tile is visible to this warp's rows (uniform per warp)

        // ---- S = Q . K^T ---------------------------------------------------------------------
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            uint32_t ah[4], al[4], b0[4], b1[4];
            const uint32_t aoff = tile_off(kQRows, a_row, 2 * ks + a_c);
            ldmatrix_x4(q_hi_s + aoff, ah[0], ah[1], ah[2], ah[3]);
            ldmatrix_x4(q_lo_s + aoff, al[0], al[1], al[2], al[3]);
            ldmatrix_x4(k_s + tile_off(kTK, bk_row, 2 * ks + bk_c), b0[0], b0[1], b0[2], b0[3]);        // positions 0..15
            ldmatrix_x4(k_s + tile_off(kTK, bk_row + 16, 2 * ks + bk_c), b1[0], b1[1], b1[2], b1[3]);   // positions 16..31
            mma16816(s[0], ah[0], ah[1], ah[2], ah[3], b0[0], b0[1]);
            mma16816(s[1], ah[0], ah[1], ah[2], ah[3], b0[2], b0[3]);
            mma16816(s[2], ah[0], ah[1], ah[2], ah[3], b1[0], b1[1]);
            mma16816(s[3], ah[0], ah[1], ah[2], ah[3], b1[2], b1[3]);
            mma16816(s[0], al[0], al[1], al[2], al[3], b0[0], b0[1]);
            mma16816(s[1], al[0], al[1], al[2], al[3], b0[2], b0[3]);
            mma16816(s[2], al[0], al[1], al[2], al[3], b1[0], b1[1]);
            mma16816(s[3], al[0], al[1], al[2], al[3], b1[2], b1[3]);
            if constexpr (!kLoTiles) continue;
            // the part of the centroids that f16 rounding dropped (a 4-bit table is only good to 1e-4)
            ldmatrix_x4(kl_s + tile_off(kTK, bk_row, 2 * ks + bk_c), b0[0], b0[1], b0[2], b0[3]);
            ldmatrix_x4(kl_s + tile_off(kTK, bk_row + 16, 2 * ks + bk_c), b1[0], b1[1], b1[2], b1[3]);
            mma16816(s[0], ah[0], ah[1], ah[2], ah[3], b0[0], b0[1]);
            mma16816(s[1], ah[0], ah[1], ah[2], ah[3], b0[2], b0[3]);
            mma16816(s[2], ah[0], ah[1], ah[2], ah[3], b1[0], b1[1]);
            mma16816(s[3], ah[0], ah[1], ah[2], ah[3], b1[2], b1[3]);
        }
        // ---- online softmax, exp2 domain; reference point = max of s + log2 ||v|| -------------
        float tv[4][4];
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int col = 8 * nt + 2 * t + e, p = pb + col;
                const float kn = sm.kn[col], lv = fast_log2(fmaxf(sm.vn[col], 1e-30f));
                const bool in = p < c1;
                s[nt][e] *= kn;
                s[nt][2 + e] *= kn;
                tv[nt][e] = (in && p < lim0) ? s[nt][e] + lv : -CUDART_INF_F;
                tv[nt][2 + e] = (in && p < lim1) ? s[nt][2 + e] + lv : -CUDART_INF_F;
                mx0 = fmaxf(mx0, tv[nt][e]);
                mx1 = fmaxf(mx1, tv[nt][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(M0, mx0), n1 = fmaxf(M1, mx1);
        // a row that has seen nothing yet keeps M = -inf; its factors must not become NaN
        const float r0 = n0 > -CUDART_INF_F ? n0 : 0.f, r1 = n1 > -CUDART_INF_F ? n1 : 0.f;
        const float f0 = fast_exp2(M0 - r0), f1 = fast_exp2(M1 - r1);  // exp2(-inf) = 0 on the first visible tile
        if (f0 != 1.f || f1 != 1.f) {
            l0 *= f0;
            l1 *= f1;
#pragma unroll
            for (int j = 0; j < 32; j++) {
                acc[j][0] *= f0;
                acc[j][1] *= f0;
                acc[j][2] *= f1;
                acc[j][3] *= f1;
            }
        }
        M0 = n0;
        M1 = n1;
        uint32_t wa[4][2], wl[4][2];  // weights as f16 pairs, hi and lo parts: [n-tile][row g | row g + 8]
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const float w00 = fast_exp2(tv[nt][0] - r0) * kWScale, w01 = fast_exp2(tv[nt][1] - r0) * kWScale;
            const float w10 = fast_exp2(tv[nt][2] - r1) * kWScale, w11 = fast_exp2(tv[nt][3] - r1) * kWScale;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (tv[nt][e] > -CUDART_INF_F) l0 += fast_exp2(s[nt][e] - r0);
                if (tv[nt][2 + e] > -CUDART_INF_F) l1 += fast_exp2(s[nt][2 + e] - r1);
            }
            const __half2 p0 = __floats2half2_rn(w00, w01), p1 = __floats2half2_rn(w10, w11);
            wa[nt][0] = *reinterpret_cast<const uint32_t *>(&p0);
            wa[nt][1] = *reinterpret_cast<const uint32_t *>(&p1);
            // a token early in the prompt sees few rows, so a single f16 weight (11 bits) would show
            const float2 f0h = __half22float2(p0), f1h = __half22float2(p1);
            const __half2 q0 = __floats2half2_rn(w00 - f0h.x, w01 - f0h.y), q1 = __floats2half2_rn(w10 - f1h.x, w11 - f1h.y);
            wl[nt][0] = *reinterpret_cast<const uint32_t *>(&q0);
            wl[nt][1] = *reinterpret_cast<const uint32_t *>(&q1);
        }
        // ---- O += W . V ------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const uint32_t a0 = wa[2 * kk][0], a1 = wa[2 * kk][1], a2 = wa[2 * kk + 1][0], a3 = wa[2 * kk + 1][1];
            const uint32_t e0 = wl[2 * kk][0], e1 = wl[2 * kk][1], e2 = wl[2 * kk + 1][0], e3 = wl[2 * kk + 1][1];
#pragma unroll
            for (int j = 0; j < 16; j++) {
                uint32_t b[4];
                ldmatrix_x4_trans(v_s + tile_off(kTK, 16 * kk + bv_row, 2 * j + bv_c), b[0], b[1], b[2], b[3]);
                mma16816(acc[2 * j], a0, a1, a2, a3, b[0], b[1]);
                mma16816(acc[2 * j + 1], a0, a1, a2, a3, b[2], b[3]);
                mma16816(acc[2 * j], e0, e1, e2, e3, b[0], b[1]);
                mma16816(acc[2 * j + 1], e0, e1, e2, e3, b[2], b[3]);
                if constexpr (!kLoTiles) continue;
                ldmatrix_x4_trans(vl_s + tile_off(kTK, 16 * kk + bv_row, 2 * j + bv_c), b[0], b[1], b[2], b[3]);
                mma16816(acc[2 * j], a0, a1, a2, a3, b[0], b[1]);
                mma16816(acc[2 * j + 1], a0, a1, a2, a3, b[2], b[3]);
            }
        }
    }

    // ---- epilogue ----------------------------------------------------------------------------
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float unscale = 1.0f / (kWScale * pa.lut_alpha);
#pragma unroll
    for (int hrow = 0; hrow < 2; hrow++) {
        const int r = hrow ? row1 : row0;
        if (r >= n_rows) continue;
        const float Mr = hrow ? M1 : M0, lr = hrow ? l1 : l0;
        const size_t out_row = (size_t)(tok0 + r / NREP) * a.n_head + kv * NREP + r % NREP;
        if (pa.n_chunks == 1) {
            const float inv = lr > 0.f ? unscale / lr : 0.f;
            float *dst = a.out + out_row * kHd;
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int d = 8 * j + 2 * t;  // a Givens pair sits in one lane
                float o0, o1;
                givens_inv(acc[j][2 * hrow] * inv, acc[j][2 * hrow + 1] * inv, sm.givens[d], sm.givens[d + 1], o0, o1);
                *reinterpret_cast<float2 *>(dst + d) = make_float2(o0, o1);
            }
        } else {
            float *dst = pa.scratch + (out_row * pa.n_chunks + chunk) * (kHd + 2);
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int d = 8 * j + 2 * t;
                *reinterpret_cast<float2 *>(dst + d) = make_float2(acc[j][2 * hrow] * unscale, acc[j][2 * hrow + 1] * unscale);
            }
            if (t == 0) {
                dst[kHd] = Mr;
                dst[kHd + 1] = lr;
            }
        }
    }
}

// One CTA of 128 threads per output row: merge the chunks' triples, rotate back, write.
__global__ void __launch_bounds__(128) prefill_merge_kernel(const float *scratch, const float *givens, int n_chunks, float *out) {
    const size_t row = blockIdx.x;
    const int pr = threadIdx.x;  // Givens pair: coordinates 2 pr, 2 pr + 1
    const float *base = scratch + row * n_chunks * (kHd + 2);
    float M = -CUDART_INF_F;
    for (int c = 0; c < n_chunks; c++) M = fmaxf(M, base[(size_t)c * (kHd + 2) + kHd]);
    float a0 = 0.f, a1 = 0.f, L = 0.f;
    for (int c = 0; c < n_chunks; c++) {
        const float *p = base + (size_t)c * (kHd + 2);
        const float m = p[kHd];
        if (!(m > -CUDART_INF_F)) continue;
        const float f = exp2f(m - M);
        const float2 v = *reinterpret_cast<const float2 *>(p + 2 * pr);
        a0 = fmaf(v.x, f, a0);
        a1 = fmaf(v.y, f, a1);
        L = fmaf(p[kHd + 1], f, L);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    float o0, o1;
    givens_inv(a0 * inv, a1 * inv, givens[2 * pr], givens[2 * pr + 1], o0, o1);
    *reinterpret_cast<float2 *>(out + row * kHd + 2 * pr) = make_float2(o0, o1);
}

template <int BITS, int NREP>
bk_status launch_prefill_one(bk_ctx *ctx, const PrefillArgs &pa) {
    static std::atomic<bool> configured[64] = {};  // per device; racing first calls set the same attribute
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, BK_ERR_UNSUPPORTED, "prefill: device index above 63");
    if (!configured[dev].load()) {
        BK_CUDA(ctx, cudaFuncSetAttribute(prefill_mma_kernel<BITS, NREP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrefillSmem));
        configured[dev].store(true);
    }
    const int grid = pa.n_blocks * pa.d.n_kv * pa.n_chunks;
    prefill_mma_kernel<BITS, NREP><<<grid, kPT, kPrefillSmem, ctx->stream>>>(pa);
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    if (pa.n_chunks > 1) {
        prefill_merge_kernel<<<pa.n_tokens * pa.d.n_head, 128, 0, ctx->stream>>>(pa.scratch, pa.d.givens, pa.n_chunks, pa.d.out);
        ctx->launches++;
        BK_CUDA(ctx, cudaGetLastError());
    }
    return BK_OK;
}

}  // namespace

bool prefill_mma_supported(const DecodeArgs &a) {
    const int n_rep = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    return a.k_kind == ROW_PLANAR && a.v_kind == ROW_PLANAR && (a.bits == 4 || a.bits == 3) &&
           (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 6);
}

// Tokens [0, n_tokens) of the call sit at cache rows pos0 .. pos0 + n_tokens - 1 (already appended).
bk_status launch_prefill_mma(bk_ctx *ctx, const DecodeArgs &a, int seq, int pos0, int n_tokens, float alpha) {
    if (n_tokens <= 0) return BK_OK;
    const int n_rep = a.n_head / a.n_kv;
    PrefillArgs pa{};
    pa.d = a;
    pa.seq = seq;
    pa.pos0 = pos0;
    pa.n_tokens = n_tokens;
    pa.tq = kQRows / n_rep;
    pa.n_blocks = (n_tokens + pa.tq - 1) / pa.tq;
    pa.lut_alpha = alpha;
    // chunks of at least 256 positions
    const int vis = pos0 + n_tokens;
    int chunks = (6 * ctx->n_sms + pa.n_blocks * a.n_kv - 1) / (pa.n_blocks * a.n_kv);  // about six CTAs per SM: the causal triangle leaves them unequal
    chunks = std::max(1, std::min(chunks, std::min(64, vis / 256)));
    pa.n_chunks = chunks;
    if (chunks > 1) {
        const size_t need = (size_t)n_tokens * a.n_head * chunks * (kHd + 2);
        if (ctx->d_prefill_floats < need) {
            BK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            if (ctx->d_prefill) cudaFree(ctx->d_prefill);
            ctx->d_prefill = nullptr;
            ctx->d_prefill_floats = 0;
            BK_CUDA(ctx, cudaMalloc((void **)&ctx->d_prefill, need * sizeof(float)));
            ctx->d_prefill_floats = need;
        }
        pa.scratch = ctx->d_prefill;
    }
#define BK_PF_CASE(R)                                                                                  \
    case R:                                                                                            \
        return a.bits == 3 ? launch_prefill_one<3, R>(ctx, pa) : launch_prefill_one<4, R>(ctx, pa);
    switch (n_rep) {
        BK_PF_CASE(1)
        BK_PF_CASE(2)
        BK_PF_CASE(4)
        BK_PF_CASE(6)
        default: return fail(ctx, BK_ERR_UNSUPPORTED, "prefill: n_head/n_kv must be 1, 2, 4 or 6");
    }
#undef BK_PF_CASE
}

}  // namespace bk
