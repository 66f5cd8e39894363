// Decode attention over a 4-bit planar cache (K and V both quantized): the bandwidth path.
//
// A 4-bit row carries 11.6 multiply-adds per byte once six q heads share it, more than the
// FP32 pipes of an SM can retire at HBM speed, and a non-uniform Lloyd-Max codebook needs a
// table lookup per index.  So this kernel
//   * reads packed rows straight into registers with 128-bit loads, two 16-position tiles
//     ahead (no shared-memory staging: the shared-memory pipe is kept for the lookups);
//   * dequantizes with one shared-memory lookup per packed BYTE: a 256-entry table of
//     half2(c[lo nibble], c[hi nibble]), replicated per lane (entry e, lane l at byte offset
//     e*256 + l*4 of a 64 KiB-aligned region) so that no lookup ever bank-conflicts and the
//     address is a single PRMT of the data byte into a per-lane base;
//   * contracts on the tensor cores with mma.sync.m16n8k16 (f16 in, f32 accumulate):
//       scores^T[16 pos x 8 heads] = Kc[16 pos x 256] . Q^T        (A = looked-up K, B = q)
//       out^T[256 x 8 heads]      += Vc^T[256 x 16 pos] . W        (A = looked-up V, B = weights)
//     The looked-up half2 registers ARE the A fragments: for K a byte holds two adjacent
//     coordinates of one position; for V the nibbles of two adjacent positions are first
//     merged into one byte so that a lookup yields one coordinate at two positions.  The
//     softmax weights move from the accumulator layout to the B layout with two movmatrix
//     transposes.  Six of the eight MMA columns are real heads (the GQA group).
// Scores and the softmax stay in f32.  The codebook is scaled by a constant alpha before
// rounding to f16 (chosen on the host so that all centroids round almost exactly); q is split
// into f16 hi + lo parts when QSPLIT is set; V weights are p * ||v|| referenced to the running
// maximum of s + log2 ||v|| and scaled by 2^14, so they use the f16 range whatever the norms.
// Output error against the f32 CPU path stays in the 1e-4 range.
//
// Work split, partials and the last-arriver combine are shared with the generic kernel.
#include <cuda_fp16.h>

#include "bk_decode_common.cuh"

namespace bk {

namespace {

constexpr int kMW = 8;                  // warps per CTA
constexpr int kMT = kMW * 32;
constexpr int kTile = 16;               // positions per warp tile (the MMA's M)
constexpr uint32_t kLutBytes = 65536;   // 256 entries x 256 B (128 B used: one word per lane)
constexpr uint32_t kOtherBytes = 10240; // q fragments + merge bookkeeping
constexpr int kHeadStride = 276;        // floats per head in the warp-merge area (bank-conflict free)
constexpr float kWScale = 16384.0f;     // 2^14: V weights are stored as f16 in (0, 2^14]
constexpr int kRowBytes = 128;          // 256 coordinates x 4 bit

struct Other {                          // lives outside the lookup table
    __half q_hi[8][kHd];
    __half q_lo[8][kHd];
    float m_w[kMW][8], l_w[kMW][8];
    float M[8], L[8];
    int last;
};
static_assert(sizeof(Other) <= kOtherBytes, "Other does not fit");

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

// Table lookup of packed byte K (0..3) of word x: lane_base holds the table's shared address in
// its upper two bytes and lane*4 in byte 0; the data byte becomes byte 1 of the address.
template <int K>
__device__ __forceinline__ uint32_t lut(uint32_t x, uint32_t lane_base) {
    uint32_t addr, v;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(addr) : "r"(x), "r"(lane_base), "n"(0x7604 | (K << 4)));
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 ldg128(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct TileRegs {
    uint4 k[4];   // K: rows g / g+8, 16-byte chunks t / t+4
    uint4 v[4];   // V: positions 2t, 2t+1, 2t+8, 2t+9, 16-byte chunk g
    float kn[2], vn[2];
};

template <int NREP, bool QSPLIT>
__global__ void __launch_bounds__(kMT, 1) decode_p4_mma_kernel(DecodeArgs a, DecodeMeta meta, float lut_alpha) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    // ---- shared-memory layout: the table must start on a 64 KiB boundary of the shared window
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t lut_addr = (base + (kLutBytes - 1)) & ~(kLutBytes - 1);
    const uint32_t other_addr = (lut_addr - base >= kOtherBytes) ? base : lut_addr + kLutBytes;
    uint8_t *lut_ptr = smem_raw + (lut_addr - base);
    Other &o = *reinterpret_cast<Other *>(smem_raw + (other_addr - base));
    const uint32_t lane_base = lut_addr | (uint32_t)(lane << 2);

    // ---- which item ------------------------------------------------------------------------
    const int item = blockIdx.x;
    int s = 0;
    while (s + 1 < meta.n_seqs && meta.item_start[s + 1] <= item) s++;
    const int n_pos = meta.n_pos[s];
    const int L = meta.chunk_len;
    const int n_chunks = (n_pos + L - 1) / L;
    const int local = item - meta.item_start[s];
    const int kv = local / n_chunks, chunk = local - kv * n_chunks;
    const int p0 = chunk * L, p1 = min(p0 + L, n_pos);
    const int n_tiles = (p1 - p0 + kTile - 1) / kTile;
    const size_t seq_rows = (size_t)meta.seq_id[s] * a.seq_stride_rows;
    const uint8_t *k_base = a.k_rows + (seq_rows + kv) * kRowBytes;
    const uint8_t *v_base = a.v_rows + (seq_rows + kv) * kRowBytes;
    const float *kn_base = a.k_norms + seq_rows + kv;
    const float *vn_base = a.v_norms + seq_rows + kv;
    const size_t row_stride = (size_t)a.n_kv * kRowBytes;

    auto load_tile = [&](int tile, TileRegs &r) {
        const int pb = p0 + tile * kTile, last = p1 - 1;
        const int pg = min(pb + g, last), pg8 = min(pb + g + 8, last);
        const uint8_t *kr0 = k_base + (size_t)pg * row_stride, *kr1 = k_base + (size_t)pg8 * row_stride;
        r.k[0] = ldg128(kr0 + t * 16);
        r.k[1] = ldg128(kr0 + (t + 4) * 16);
        r.k[2] = ldg128(kr1 + t * 16);
        r.k[3] = ldg128(kr1 + (t + 4) * 16);
        const int pv0 = min(pb + 2 * t, last), pv1 = min(pb + 2 * t + 1, last);
        const int pv2 = min(pb + 2 * t + 8, last), pv3 = min(pb + 2 * t + 9, last);
        r.v[0] = ldg128(v_base + (size_t)pv0 * row_stride + g * 16);
        r.v[1] = ldg128(v_base + (size_t)pv1 * row_stride + g * 16);
        r.v[2] = ldg128(v_base + (size_t)pv2 * row_stride + g * 16);
        r.v[3] = ldg128(v_base + (size_t)pv3 * row_stride + g * 16);
        r.kn[0] = __ldg(kn_base + (size_t)pg * a.n_kv);
        r.kn[1] = __ldg(kn_base + (size_t)pg8 * a.n_kv);
        r.vn[0] = __ldg(vn_base + (size_t)pg * a.n_kv);
        r.vn[1] = __ldg(vn_base + (size_t)pg8 * a.n_kv);
    };

    TileRegs buf0, buf1;
    if (warp < n_tiles) load_tile(warp, buf0);
    if (warp + kMW < n_tiles) load_tile(warp + kMW, buf1);

    // ---- q: rope, Givens rotation, scale, split into f16 hi/lo (scratch: the table's region) --
    {
        float *sq = reinterpret_cast<float *>(lut_ptr);  // [NREP][256]
        const float *q = a.q + ((size_t)meta.slot[s] * a.n_head + (size_t)kv * NREP) * kHd;
        for (int i = tid; i < NREP * kHd; i += kMT) sq[i] = q[i];
        __syncthreads();
        if (!a.no_rope) {
            const int half = a.n_rot >> 1;
            const float2 *cs = a.rope + (size_t)meta.q_pos[s] * half;
            for (int i = tid; i < NREP * half; i += kMT) {
                const int r = i / half, j = i - r * half;
                float x0 = sq[r * kHd + j], x1 = sq[r * kHd + j + half];
                rope_pair(x0, x1, cs[j]);
                sq[r * kHd + j] = x0;
                sq[r * kHd + j + half] = x1;
            }
            __syncthreads();
        }
        // 1/sqrt(hd) * log2(e) / alpha: the scores come out in the exp2 domain, alpha undone
        const float qscale = rsqrtf((float)kHd) * 1.4426950408889634f / lut_alpha;
        for (int i = tid; i < 8 * (kHd / 2); i += kMT) {
            const int r = i / (kHd / 2), pr = i - r * (kHd / 2);
            float o0 = 0.f, o1 = 0.f;
            if (r < NREP) {
                givens_fwd(sq[r * kHd + 2 * pr], sq[r * kHd + 2 * pr + 1], a.givens[2 * pr], a.givens[2 * pr + 1], o0, o1);
                o0 *= qscale;
                o1 *= qscale;
            }
            const __half h0 = __float2half_rn(o0), h1 = __float2half_rn(o1);
            o.q_hi[r][2 * pr] = h0;
            o.q_hi[r][2 * pr + 1] = h1;
            o.q_lo[r][2 * pr] = __float2half_rn(o0 - __half2float(h0));
            o.q_lo[r][2 * pr + 1] = __float2half_rn(o1 - __half2float(h1));
        }
        __syncthreads();
    }
    // ---- the lookup table: entry e -> half2(alpha*c[e & 15], alpha*c[e >> 4]), one copy per lane
    {
        const float c_lo = a.book[lane & 15] * lut_alpha;  // lanes 0..15 hold the 16 scaled centroids
        for (int e = warp; e < 256; e += kMW) {
            const float lo = __shfl_sync(0xffffffffu, c_lo, e & 15), hi = __shfl_sync(0xffffffffu, c_lo, e >> 4);
            const __half2 h = __floats2half2_rn(lo, hi);
            *reinterpret_cast<__half2 *>(lut_ptr + e * 256 + lane * 4) = h;
        }
        __syncthreads();
    }

    // ---- q fragments: k-step ks = c*8 + w*2 + bp covers coordinates (t+4c)*32 + w*8 + bp*4 + 0..3
    uint32_t qh[16][2];
#pragma unroll
    for (int ks = 0; ks < 16; ks++) {
        const int c = ks >> 3, w = (ks >> 1) & 3, bp = ks & 1;
        const int d0 = (t + 4 * c) * 32 + w * 8 + bp * 4;
        const uint2 v = *reinterpret_cast<const uint2 *>(&o.q_hi[g][d0]);
        qh[ks][0] = v.x;
        qh[ks][1] = v.y;
    }
    uint32_t ql[QSPLIT ? 16 : 1][2];
    if (QSPLIT) {
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            const int c = ks >> 3, w = (ks >> 1) & 3, bp = ks & 1;
            const int d0 = (t + 4 * c) * 32 + w * 8 + bp * 4;
            const uint2 v = *reinterpret_cast<const uint2 *>(&o.q_lo[g][d0]);
            ql[QSPLIT ? ks : 0][0] = v.x;
            ql[QSPLIT ? ks : 0][1] = v.y;
        }
    }

    float acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    float M0 = -CUDART_INF_F, M1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    const int dbg = a.dbg;
    auto compute_tile = [&](int tile, const TileRegs &r) {
        // ---- scores^T = Kc . Q^T ------------------------------------------------------------
        // four independent accumulator chains (the 16 or 32 MMAs of a tile would otherwise be one
        // dependent chain), summed at the end
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
        float sc2[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
        if (!(dbg & 2))
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint32_t xg[4] = {r.k[c].x, r.k[c].y, r.k[c].z, r.k[c].w};
            const uint32_t xh[4] = {r.k[2 + c].x, r.k[2 + c].y, r.k[2 + c].z, r.k[2 + c].w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const int ks = c * 8 + w * 2;
                {
                    const uint32_t a0 = lut<0>(xg[w], lane_base), a1 = lut<0>(xh[w], lane_base);
                    const uint32_t a2 = lut<1>(xg[w], lane_base), a3 = lut<1>(xh[w], lane_base);
                    mma16816(c ? sb : sa, a0, a1, a2, a3, qh[ks][0], qh[ks][1]);
                    if (QSPLIT) mma16816(c ? sd : sc2, a0, a1, a2, a3, ql[QSPLIT ? ks : 0][0], ql[QSPLIT ? ks : 0][1]);
                }
                {
                    const uint32_t a0 = lut<2>(xg[w], lane_base), a1 = lut<2>(xh[w], lane_base);
                    const uint32_t a2 = lut<3>(xg[w], lane_base), a3 = lut<3>(xh[w], lane_base);
                    mma16816(c ? sd : sc2, a0, a1, a2, a3, qh[ks + 1][0], qh[ks + 1][1]);
                    if (QSPLIT) mma16816(c ? sb : sa, a0, a1, a2, a3, ql[QSPLIT ? ks + 1 : 0][0], ql[QSPLIT ? ks + 1 : 0][1]);
                }
            }
        }
        float sc[4];
#pragma unroll
        for (int i = 0; i < 4; i++) sc[i] = (sa[i] + sb[i]) + (sc2[i] + sd[i]);
        // ---- online softmax in the exp2 domain; reference point = max of s + log2||v|| -------
        const int pb = p0 + tile * kTile;
        const bool ok0 = pb + g < p1, ok1 = pb + g + 8 < p1;
        const float s00 = sc[0] * r.kn[0], s01 = sc[1] * r.kn[0], s10 = sc[2] * r.kn[1], s11 = sc[3] * r.kn[1];
        const float lv0 = log2f(fmaxf(r.vn[0], 1e-37f)), lv1 = log2f(fmaxf(r.vn[1], 1e-37f));
        const float t00 = ok0 ? s00 + lv0 : -CUDART_INF_F, t01 = ok0 ? s01 + lv0 : -CUDART_INF_F;
        const float t10 = ok1 ? s10 + lv1 : -CUDART_INF_F, t11 = ok1 ? s11 + lv1 : -CUDART_INF_F;
        float mx0 = fmaxf(t00, t10), mx1 = fmaxf(t01, t11);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const bool grow = (mx0 > M0) || (mx1 > M1);
        if (__any_sync(0xffffffffu, grow)) {
            const float n0 = fmaxf(M0, mx0), n1 = fmaxf(M1, mx1);
            const float c0 = exp2f(M0 - n0), c1 = exp2f(M1 - n1);  // 0 on the first tile
            l0 *= c0;
            l1 *= c1;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                acc[j][0] *= c0;
                acc[j][1] *= c1;
                acc[j][2] *= c0;
                acc[j][3] *= c1;
            }
            M0 = n0;
            M1 = n1;
        }
        const float w00 = exp2f(t00 - M0) * kWScale, w01 = exp2f(t01 - M1) * kWScale;
        const float w10 = exp2f(t10 - M0) * kWScale, w11 = exp2f(t11 - M1) * kWScale;
        l0 += (ok0 ? exp2f(s00 - M0) : 0.f) + (ok1 ? exp2f(s10 - M0) : 0.f);
        l1 += (ok0 ? exp2f(s01 - M1) : 0.f) + (ok1 ? exp2f(s11 - M1) : 0.f);
        const __half2 pl = __floats2half2_rn(w00, w01), ph = __floats2half2_rn(w10, w11);
        const uint32_t b0 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&pl));  // head g; pos 2t, 2t+1
        const uint32_t b1 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph));  // head g; pos 2t+8, 2t+9
        // ---- out^T += Vc^T . W : MMA j covers coordinates 32g + 2j (rows g) and 32g + 2j + 1 (rows g+8)
        const uint32_t x0[4] = {r.v[0].x, r.v[0].y, r.v[0].z, r.v[0].w};
        const uint32_t x1[4] = {r.v[1].x, r.v[1].y, r.v[1].z, r.v[1].w};
        const uint32_t x2[4] = {r.v[2].x, r.v[2].y, r.v[2].z, r.v[2].w};
        const uint32_t x3[4] = {r.v[3].x, r.v[3].y, r.v[3].z, r.v[3].w};
        if (!(dbg & 4))
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t m = 0x0f0f0f0fu;
            const uint32_t lo01 = (x0[w] & m) | ((x1[w] & m) << 4), hi01 = ((x0[w] >> 4) & m) | (x1[w] & ~m);
            const uint32_t lo23 = (x2[w] & m) | ((x3[w] & m) << 4), hi23 = ((x2[w] >> 4) & m) | (x3[w] & ~m);
            mma16816(acc[4 * w + 0], lut<0>(lo01, lane_base), lut<0>(hi01, lane_base), lut<0>(lo23, lane_base),
                     lut<0>(hi23, lane_base), b0, b1);
            mma16816(acc[4 * w + 1], lut<1>(lo01, lane_base), lut<1>(hi01, lane_base), lut<1>(lo23, lane_base),
                     lut<1>(hi23, lane_base), b0, b1);
            mma16816(acc[4 * w + 2], lut<2>(lo01, lane_base), lut<2>(hi01, lane_base), lut<2>(lo23, lane_base),
                     lut<2>(hi23, lane_base), b0, b1);
            mma16816(acc[4 * w + 3], lut<3>(lo01, lane_base), lut<3>(hi01, lane_base), lut<3>(lo23, lane_base),
                     lut<3>(hi23, lane_base), b0, b1);
        }
    };

    // ---- scan: two tiles in flight per warp ----------------------------------------------------
    for (int tile = warp; tile < n_tiles; tile += 2 * kMW) {
        compute_tile(tile, buf0);
        if (tile + 2 * kMW < n_tiles) load_tile(tile + 2 * kMW, buf0);
        if (tile + kMW < n_tiles) {
            compute_tile(tile + kMW, buf1);
            if (tile + 3 * kMW < n_tiles) load_tile(tile + 3 * kMW, buf1);
        }
    }

    if (dbg & 1) { if (M0 == 123.f) a.out[0] = l0 + acc[0][0] + acc[5][1]; return; }
    // ---- merge the warps ---------------------------------------------------------------------
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    if (g == 0) {
        o.m_w[warp][2 * t] = M0;
        o.m_w[warp][2 * t + 1] = M1;
        o.l_w[warp][2 * t] = l0;
        o.l_w[warp][2 * t + 1] = l1;
    }
    __syncthreads();  // every warp is also done with the lookup table
    if (tid < 8) {
        float M = -CUDART_INF_F;
        for (int w = 0; w < kMW; w++) M = fmaxf(M, o.m_w[w][tid]);
        float Ls = 0.f;
        for (int w = 0; w < kMW; w++)
            if (o.m_w[w][tid] > -CUDART_INF_F) Ls += o.l_w[w][tid] * exp2f(o.m_w[w][tid] - M);
        o.M[tid] = M;
        o.L[tid] = Ls;
    }
    __syncthreads();
    float *area = reinterpret_cast<float *>(lut_ptr);  // [kMW][NREP][kHeadStride], reuses the table
    {
        const float unscale = 1.0f / (kWScale * lut_alpha);
        const float f0 = (M0 > -CUDART_INF_F) ? exp2f(M0 - o.M[2 * t]) * unscale : 0.f;
        const float f1 = (M1 > -CUDART_INF_F) ? exp2f(M1 - o.M[2 * t + 1]) * unscale : 0.f;
        float *w0 = area + ((size_t)warp * NREP + 2 * t) * kHeadStride + g * 33;
        float *w1 = w0 + kHeadStride;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if (2 * t < NREP) {
                w0[2 * j] = acc[j][0] * f0;
                w0[2 * j + 1] = acc[j][2] * f0;
            }
            if (2 * t + 1 < NREP) {
                w1[2 * j] = acc[j][1] * f1;
                w1[2 * j + 1] = acc[j][3] * f1;
            }
        }
    }
    __syncthreads();
    float sums[NREP];
    {
        const int d = tid, idx = d + (d >> 5);  // coordinate d sits at g*33 + (d & 31), g = d >> 5
#pragma unroll
        for (int r = 0; r < NREP; r++) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kMW; w++) sum += area[((size_t)w * NREP + r) * kHeadStride + idx];
            sums[r] = sum;
        }
    }
    __syncthreads();
    float *s_acc = area;  // [NREP][256]
#pragma unroll
    for (int r = 0; r < NREP; r++) s_acc[r * kHd + tid] = sums[r];
    __syncthreads();

    if (dbg & 8) return;
    const int first_item = meta.item_start[s] + kv * n_chunks;
    finish_item<NREP>(a, meta.slot[s], s, kv, item, n_chunks, first_item, s_acc, o.M, o.L, &o.last, true);
}

template <int NREP, bool QSPLIT>
bk_status launch_one(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float alpha) {
    const size_t smem = 2 * (size_t)kLutBytes + kOtherBytes;
    static bool configured[64] = {};  // per template instance and device
    if (ctx->device >= 64 || !configured[ctx->device]) {
        cudaError_t e = cudaFuncSetAttribute(decode_p4_mma_kernel<NREP, QSPLIT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(decode_p4_mma_kernel)");
        if (ctx->device < 64) configured[ctx->device] = true;
    }
    decode_p4_mma_kernel<NREP, QSPLIT><<<m.n_items, kMT, smem, ctx->stream>>>(a, m, alpha);
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace

bool decode_mma_supported(const DecodeArgs &a) {
    const int n_rep = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    return a.k_kind == ROW_PLANAR && a.v_kind == ROW_PLANAR && a.bits == 4 &&
           (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 6);
}

bk_status launch_decode_mma(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float alpha, bool qsplit) {
    if (m.n_items <= 0) return BK_OK;
    const int n_rep = a.n_head / a.n_kv;
#define BK_MMA_CASE(R)                                                          \
    case R:                                                                     \
        return qsplit ? launch_one<R, true>(ctx, a, m, alpha) : launch_one<R, false>(ctx, a, m, alpha);
    switch (n_rep) {
        BK_MMA_CASE(1)
        BK_MMA_CASE(2)
        BK_MMA_CASE(4)
        BK_MMA_CASE(6)
        default: return fail(ctx, BK_ERR_UNSUPPORTED, "decode (mma): n_head/n_kv must be 1, 2, 4 or 6");
    }
#undef BK_MMA_CASE
}

}  // namespace bk
