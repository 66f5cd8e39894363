// Decode attention over a 4-bit (or 3-bit, or 2-bit) planar cache (K and V both quantized): the bandwidth path.
//
// A 4-bit row carries 11.6 multiply-adds per byte once six q heads share it, more than the
// FP32 pipes of an SM can retire at HBM speed, and a non-uniform Lloyd-Max codebook needs a
// table lookup per index.  So this kernel
//   * streams packed rows through a per-warp ring of shared-memory stages filled by the TMA
//     engine: one tiled cp.async.bulk.tensor copy of 32 rows x 128 bytes for K and one for V per
//     tile (a 3-D tensor map over [position][kv head][128 B] picks the rows of one kv head out
//     of the interleaved cache) plus two small plain bulk copies for the norms of the same 32
//     positions, completion on an mbarrier with a bounded wait.  HBM latency
//     on this part needs more than 100 KB in flight per SM, which registers cannot hold.  The
//     tiles land with the 128-byte swizzle (16-byte chunk ^= row & 7), and the kernel reads
//     K as (row g, chunks 2t, 2t+1) and V as (rows 2t.., chunk g), which makes every 128-bit
//     fragment read conflict-free;
//   * dequantizes with one shared-memory lookup per packed BYTE: a 256-entry table of
//     half2(c[lo nibble], c[hi nibble]), replicated per lane (entry e, lane l at byte offset
//     e*256 + l*4 of a 64 KiB-aligned region) so that no lookup ever bank-conflicts and the
//     address is a single PRMT of the data byte into a per-lane base;
//   * contracts on the tensor cores with mma.sync.m16n8k16 (f16 in, f32 accumulate), two row
//     blocks of 16 positions per step so that every dependent chain has an independent twin:
//       scores^T[16 pos x 8 heads] = Kc[16 pos x 256] . Q^T        (A = looked-up K, B = q)
//       out^T[256 x 8 heads]      += Vc^T[256 x 16 pos] . W        (A = looked-up V, B = weights)
//     The looked-up half2 registers ARE the A fragments: for K a byte holds two adjacent
//     coordinates of one position; for V the nibbles of two adjacent positions are first
//     merged into one byte so that a lookup yields one coordinate at two positions.  The
//     softmax weights move from the accumulator layout to the B layout with two movmatrix
//     transposes.  Six of the eight MMA columns are real heads (the GQA group);
//   * keeps q in registers as B fragments (prepared once by the whole CTA through shared memory):
//     no shared-memory read of q in the scan, and from the start of the scan to its end no warp
//     waits for another one.
// Scores and the softmax stay in f32.  The codebook is scaled by a constant alpha before
// rounding to f16 (chosen on the host so that all centroids round almost exactly); q is split
// into f16 hi + lo parts when QSPLIT is set; V weights are p * ||v|| referenced to the running
// maximum of s + log2 ||v|| and scaled by 2^14, so they use the f16 range whatever the norms.
// Output error against the f32 CPU path stays in the 1e-4 range.
//
// Work split.  A launch has about one CTA (8 warps) per SM; a CTA owns a contiguous chunk of one
// (sequence, kv head) - contiguous chunks stream measurably faster than interleaved ones - and
// its warps take the chunk's tiles in fixed shares (the result then does not depend on timing);
// in the CTA of the last chunk the two warps that first store the new token's rows (the fused
// append) join after a head start of the others.  BONSAI_KV_DYN=1 lets the warps draw tiles from
// a counter in shared memory instead (same speed on an idle GPU, results vary in the last bits).
// Partials and the split-K combine are shared with the other decode kernels.
#include <cuda.h>
#include <cuda_fp16.h>

#include <atomic>

#include "bk_decode_common.cuh"
#include "bk_mma_common.cuh"

namespace bk {

namespace {

constexpr int kMW = 8;                  // warps per CTA (two per scheduler, up to 255 registers each)
constexpr int kMT = kMW * 32;
constexpr int kTile = 32;               // positions per warp tile: two MMA row blocks of 16
constexpr uint32_t kLutBytes = 65536;   // 256 entries x 256 B (128 B used: one word per lane)
constexpr int kHeadStride = 276;        // floats per head in the warp-merge area (bank-conflict free)
constexpr float kWScale = 16384.0f;     // 2^14: V weights are stored as f16 in (0, 2^14]
constexpr int kMaxStages = 4;
// Per index width (4, 3 or 2 bits): a row is 32 * BITS bytes, a tile 32 dense rows (4-bit tiles land
// with the 128-byte swizzle, 2-bit tiles with the 64-byte one, 3-bit tiles plain; 3- and 2-bit indices are
// widened to nibbles before the table lookups), a stage = K tile, V tile, K norms, V norms (the
// norms of every kv head travel: 32 positions x n_kv floats, padded to 512 or 1024 bytes).
template <int BITS> struct Width {
    static constexpr int kRowBytes = 32 * BITS;
    static constexpr int kTileBytes = kTile * kRowBytes;  // 4096 / 3072
};
// Which shared-memory row holds the MMA's position row g.  4 bit: g itself (the swizzle spreads
// the banks).  3 bit: rows are 96 bytes apart and unswizzled; this order makes both the K reads
// (row g, 8 bytes at 24 t) and the V reads (rows 2t, 2t+1, 4 bytes at 12 g) spread over the banks.
// 2 bit: rows are 64 bytes apart and land with the 64-byte swizzle (16-byte chunk ^= (row >> 1) & 3); this order
// gives the K reads (row g, chunk t) two rows of different parity per quarter warp and the V reads (rows 2t,
// 2t + 1, 8 bytes at 8 g) four rows with different (row & 1, row & 4): both conflict-free.
template <int BITS> __device__ __forceinline__ int row_of(int g) {
    if constexpr (BITS == 3) return (g < 4) ? g : (g ^ 1);  // 0 1 2 3 5 4 7 6
    else if constexpr (BITS == 2) return ((0x65742130u >> (4 * g)) & 7);  // 0 3 1 2 4 7 5 6
    else return g;
}
// Eight 3-bit indices in the low 24 bits of y -> eight nibbles.
__device__ __forceinline__ uint32_t expand24(uint32_t y) {
    y &= 0x00ffffffu;
    y += (y & 0x00fff000u) * 15u;   // upper four indices up by 4 bits
    y += (y & 0x0fc00fc0u) * 3u;    // upper two of every four up by 2
    y += (y & 0x38383838u);         // upper one of every two up by 1
    return y;
}
// Eight 2-bit indices in the low 16 bits of y -> eight nibbles.
__device__ __forceinline__ uint32_t expand16(uint32_t y) {
    y &= 0x0000ffffu;
    y = (y | (y << 8)) & 0x00ff00ffu;
    y = (y | (y << 4)) & 0x0f0f0f0fu;
    y = (y | (y << 2)) & 0x33333333u;
    return y;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

struct Other {                          // bookkeeping block, lives outside the lookup table
    float givens[kHd];                   // (cos, sin) pairs
    float2 rope_row[kHd / 2];            // (cos, sin) of the q position
    float qw[kHd];                       // q RMSNorm weight (layer form of the step)
    float new_row[2][kHd];               // the newest token's k and v of this kv head (fused append)
    float book[2][16];                   // unscaled centroids, one copy per appending warp
    float m_w[kMW][8], l_w[kMW][8];
    float M[8], L[8];
    int last;
    int next_tile;                       // the chunk's tile counter
    unsigned long long bar[kMW][kMaxStages];  // one mbarrier per warp and stage
    unsigned long long fin_bar[2];            // the split-K combine's two streaming rounds
};
constexpr uint32_t kOtherBytes = 7168;
static_assert(sizeof(Other) <= kOtherBytes, "Other does not fit");

// Table lookup of packed byte K (0..3) of word x: lane_base holds the table's shared address in
// its upper two bytes and lane*4 in byte 0; the data byte becomes byte 1 of the address.
template <int K>
__device__ __forceinline__ uint32_t lut(uint32_t x, uint32_t lane_base) {
    uint32_t addr, v;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(addr) : "r"(x), "r"(lane_base), "n"(0x7604 | (K << 4)));
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

// The same lookup with the entry's rounding remainder (the upper half of the table slot, see PRECISE).
template <int K>
__device__ __forceinline__ void lut2(uint32_t x, uint32_t lane_base, uint32_t &v, uint32_t &rem) {
    uint32_t addr;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(addr) : "r"(x), "r"(lane_base), "n"(0x7604 | (K << 4)));
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    asm volatile("ld.shared.b32 %0, [%1+128];\n" : "=r"(rem) : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
    return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

template <int BITS, int NREP, bool QSPLIT, bool PRECISE = false>
__global__ void __launch_bounds__(kMT, 1)
decode_p4_mma_kernel(DecodeArgs a, DecodeMeta meta, float lut_alpha, uint32_t smem_bytes, int *err_flag,
                     const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    constexpr int kRowBytes = Width<BITS>::kRowBytes, kTileBytes = Width<BITS>::kTileBytes;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    // ---- shared-memory layout.  The table must start on a 64 KiB boundary of the shared window
    // (its index is spliced into byte 1 of the address).  The bookkeeping block sits at the very
    // end of the window; what lies before the table and between the table and that block holds the
    // per-warp stage ring; the number of stages is whatever fits.
    const uint32_t nb = (uint32_t)(kTile * 4 * a.n_kv);      // norms of 32 positions, every kv head
    const uint32_t norm_pad = (nb + 511u) & ~511u;
    const uint32_t stage_bytes = 2 * kTileBytes + 2 * norm_pad;  // a multiple of 1 KiB
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t lut_addr = (base + (kLutBytes - 1)) & ~(kLutBytes - 1);
    const uint32_t other_addr = (base + smem_bytes - kOtherBytes) & ~15u;
    const uint32_t a_lo = (base + 1023u) & ~1023u, a_hi = lut_addr;      // region before the table
    const uint32_t b_lo = lut_addr + kLutBytes, b_hi = other_addr;      // region after it
    const uint32_t n_a = (a_hi > a_lo ? a_hi - a_lo : 0u) / stage_bytes, n_b = (b_hi > b_lo ? b_hi - b_lo : 0u) / stage_bytes;
    const int n_stages = min((int)((n_a + n_b) / kMW), kMaxStages);
    if (n_stages < 1 || b_lo > b_hi) {  // the table's alignment left no room for the ring: report, do not run
        if (tid == 0) raise_error(err_flag, 2);
        asm volatile("griddepcontrol.wait;\n" ::: "memory");  // keep the stream's kernel order intact
        return;
    }
    auto stage_addr = [&](int st) -> uint32_t {
        const uint32_t n = (uint32_t)(warp * n_stages + st);
        return n < n_a ? a_lo + n * stage_bytes : b_lo + (n - n_a) * stage_bytes;
    };
    uint8_t *lut_ptr = smem_raw + (lut_addr - base);
    Other &o = *reinterpret_cast<Other *>(smem_raw + (other_addr - base));
    const uint32_t lane_base = lut_addr | (uint32_t)(lane << 2);
    const uint32_t bar0 = other_addr + (uint32_t)offsetof(Other, bar) + (uint32_t)(warp * kMaxStages) * 8u;
    if (lane < kMaxStages) mbar_init(bar0 + lane * 8u, 1);
    if (tid < 2) mbar_init(other_addr + (uint32_t)offsetof(Other, fin_bar) + tid * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");

    // ---- which item ------------------------------------------------------------------------
    const int item = blockIdx.x;
    int s = 0;
    while (s + 1 < meta.n_seqs && meta.item_start[s + 1] <= item) s++;
    const int n_pos = meta.n_pos[s];
    const int L = meta.chunk_len;  // a multiple of 128 positions
    const int n_chunks = (n_pos + L - 1) / L;
    const int local = item - meta.item_start[s];
    const int kv = local / n_chunks, chunk = local - kv * n_chunks;
    const int p0 = chunk * L, p1 = min(p0 + L, n_pos);
    const int tile0 = p0 / kTile;                              // first tile of the chunk (sequence-wide index)
    const bool appender = a.new_k != nullptr && chunk == n_chunks - 1;
    // The tile that holds the new token's row is not drawn from the pool: warp 0 of the appending
    // CTA takes it once that row is stored.
    const int n_tiles = (p1 - p0 + kTile - 1) / kTile, n_pool = n_tiles - (appender ? 1 : 0);
    const size_t seq_rows = (size_t)meta.seq_id[s] * a.seq_stride_rows;
    const bool dyn = (a.dyn & 1) != 0;

    // One lane arms the stage's mbarrier and issues the tile's four copies.  Rows past the end of
    // the sequence are whatever follows in the cache (or zeros past its end); their weights are
    // forced to zero below.
    const int gpos0 = a.layer_pos0 + meta.seq_id[s] * a.n_ctx;  // position index in the tensor map
    uint32_t st_base[kMaxStages];  // this warp's stage addresses
#pragma unroll
    for (int i = 0; i < kMaxStages; i++) st_base[i] = stage_addr(i < n_stages ? i : 0);
    auto stage_of = [&](int st) -> uint32_t {
        uint32_t r = st_base[0];
#pragma unroll
        for (int i = 1; i < kMaxStages; i++) r = (st == i) ? st_base[i] : r;
        return r;
    };
    const float *kn_src = a.k_norms + seq_rows, *vn_src = a.v_norms + seq_rows;
    auto issue_tile = [&](int lt, int st) {  // lt: tile index inside the chunk
        if (lane == 0) {
            const int pos = (tile0 + lt) * kTile;
            const uint32_t bar = bar0 + (uint32_t)st * 8u, dst = stage_of(st);
            mbar_expect_tx(bar, 2 * kTileBytes + 2 * nb);
            tma_tile(dst, &tm_k, kv, gpos0 + pos, bar);
            tma_tile(dst + kTileBytes, &tm_v, kv, gpos0 + pos, bar);
            const uint32_t noff = (uint32_t)(pos * a.n_kv);
            tma_bulk(dst + 2 * kTileBytes, kn_src + noff, nb, bar);
            tma_bulk(dst + 2 * kTileBytes + norm_pad, vn_src + noff, nb, bar);
        }
    };
    auto wait_tile = [&](int st, uint32_t parity) {
        const uint32_t bar = bar0 + (uint32_t)st * 8u;
        int polls = 0;
        while (!mbar_try_wait(bar, parity)) {
            if (++polls > kWaitPolls) {  // never expected; leave a mark and go on rather than hang
                if (lane == 0) raise_error(err_flag, 1);
                break;
            }
        }
    };
    // ---- set-up that touches only constant tables comes first: with programmatic dependent launch
    // it overlaps the tail of the previous kernel in the stream.  Everything a previous kernel may
    // have written (q, the newest cache row, the split-K scratch) is read after the wait below.
    {
        for (int i = tid; i < kHd; i += kMT) o.givens[i] = a.givens[i];
        if (!a.no_rope) {
            const int half = a.n_rot >> 1;
            const float2 *cs = a.rope + (size_t)meta.q_pos[s] * half;
            for (int i = tid; i < half; i += kMT) o.rope_row[i] = cs[i];
        }
        if (a.q_norm_w)
            for (int i = tid; i < kHd; i += kMT) o.qw[i] = a.q_norm_w[i];
        if (tid < 2 * 16) o.book[tid >> 4][tid & 15] = (tid & 15) < (1 << BITS) ? a.book[tid & 15] : 0.f;
        if (tid == 0) o.next_tile = kMW * n_stages;  // the first n_stages tiles of every warp are fixed
        constexpr int kIdxMask = (1 << BITS) - 1;
        const float c_lo = a.book[lane & kIdxMask] * lut_alpha;  // the low lanes hold the scaled centroids
        // the lookup table: entry e -> half2(alpha*c[low nibble], alpha*c[high nibble]), one copy per lane
        for (int e = warp; e < 256; e += kMW) {
            const float lo = __shfl_sync(0xffffffffu, c_lo, e & kIdxMask), hi = __shfl_sync(0xffffffffu, c_lo, (e >> 4) & kIdxMask);
            const __half2 h = __floats2half2_rn(lo, hi);
            *reinterpret_cast<__half2 *>(lut_ptr + e * 256 + lane * 4) = h;
        }
    }
    __syncthreads();  // tables and barriers are ready; from here to the end of the scan the warps run on their own
    BK_STAMP(0);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    BK_STAMP(1);
    // the counter set of the next launch: whatever the launch before the previous one left there goes now
    if (blockIdx.x == 0 && a.counters_other)
        for (int i = tid; i < a.other_n; i += blockDim.x) a.counters_other[i] = 0;


    // ---- q first: its loads are in flight before the tile copies fill the memory system's queues
    constexpr int kQPer = (NREP * kHd + kMT - 1) / kMT;
    float q_reg[kQPer];
    {
        const float *q = a.q + ((size_t)meta.slot[s] * a.n_head + (size_t)kv * NREP) * a.q_stride;
#pragma unroll
        for (int u = 0; u < kQPer; u++) {
            const int i = tid + u * kMT;
            q_reg[u] = i < NREP * kHd ? __ldg(q + (size_t)(i >> 8) * a.q_stride + (i & 255)) : 0.f;
        }
    }
    // Fixed shares (the default: the result then does not depend on timing).  Warp w takes tiles w, w + 8, ...;
    // in the appending CTA warps 0 and 1 start late (they store the new rows first), so there the other six
    // warps share the first kHeadStart rounds among themselves.
    constexpr int kHeadStart = 4;
    auto fixed_tile = [&](int i) -> int {
        if (!appender) return warp + kMW * i;
        if (warp < 2) return (kMW - 2) * kHeadStart + kMW * i + warp;
        return i < kHeadStart ? (kMW - 2) * i + (warp - 2) : (kMW - 2) * kHeadStart + kMW * (i - kHeadStart) + warp;
    };
    // ---- fill the ring
    int in_stage[kMaxStages];  // which tile each stage holds, -1 = none
#pragma unroll
    for (int st = 0; st < kMaxStages; st++) {
        const int lt = dyn ? warp + st * kMW : fixed_tile(st);
        in_stage[st] = (st < n_stages && lt < n_pool) ? lt : -1;
        if (in_stage[st] >= 0) issue_tile(lt, st);
    }
    int i_next = n_stages;
    // ---- q: per-head RMSNorm (layer form), rope, Givens rotation, scale, split into f16 hi/lo, written in the
    // MMA's B-fragment layout and then fetched by every lane into registers.  The scratch for this is the
    // unused upper half of the table's 256-byte slots (the table itself fills only the lower halves):
    // slot h, word x is at table + 256 h + 128 + 4 x.  sq[i] takes slots 0..47, the fragments slots 64..127.
    uint32_t qh[16][2], ql[QSPLIT ? 16 : 1][2];
    {
        auto sq = [&](int i) -> float & { return *reinterpret_cast<float *>(lut_ptr + (i >> 5) * 256 + 128 + (i & 31) * 4); };
        auto frag = [&](int lo_part, int j) -> uint2 & {  // j = k-step * 32 + lane
            return *reinterpret_cast<uint2 *>(lut_ptr + (64 + 32 * lo_part + (j >> 4)) * 256 + 128 + (j & 15) * 8);
        };
#pragma unroll
        for (int u = 0; u < kQPer; u++) {
            const int i = tid + u * kMT;
            if (i < NREP * kHd) sq(i) = q_reg[u];
        }
        __syncthreads();
        if (a.q_norm_w) {  // per-head RMSNorm of q (src/forward.rs:242-243); q is not stored, so a tree sum will do
            if (warp < NREP) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < kHd / 32; j++) {
                    const float x = sq(warp * kHd + lane + 32 * j);
                    ss = fmaf(x, x, ss);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                if (lane == 0) o.M[warp] = 1.0f / sqrtf(ss / (float)kHd + a.eps);
            }
            __syncthreads();
            for (int i = tid; i < NREP * kHd; i += kMT) sq(i) = sq(i) * o.M[i >> 8] * o.qw[i & 255];
            __syncthreads();
        }
        if (!a.no_rope) {
            const int half = a.n_rot >> 1;
            for (int i = tid; i < NREP * half; i += kMT) {
                const int r = i / half, j = i - r * half;
                float x0 = sq(r * kHd + j), x1 = sq(r * kHd + j + half);
                rope_pair(x0, x1, o.rope_row[j]);
                sq(r * kHd + j) = x0;
                sq(r * kHd + j + half) = x1;
            }
            __syncthreads();
        }
        // 1/sqrt(hd) * log2(e) / alpha: the scores come out in the exp2 domain, alpha undone.
        // k-step ks = c*8 + w*2 + bp covers coordinates (2t+c)*32 + w*8 + bp*4 + 0..3 of head g.
        const float qscale = rsqrtf((float)kHd) * 1.4426950408889634f / lut_alpha;
        for (int i = tid; i < 16 * 32; i += kMT) {
            const int ks = i >> 5, ln = i & 31, gg = ln >> 2, tt = ln & 3;
            const int c = ks >> 3, w = (ks >> 1) & 3, bp = ks & 1;
            const int d0 = (2 * tt + c) * 32 + w * 8 + bp * 4;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (gg < NREP) {
                givens_fwd(sq(gg * kHd + d0), sq(gg * kHd + d0 + 1), o.givens[d0], o.givens[d0 + 1], x[0], x[1]);
                givens_fwd(sq(gg * kHd + d0 + 2), sq(gg * kHd + d0 + 3), o.givens[d0 + 2], o.givens[d0 + 3], x[2], x[3]);
            }
            __half h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                x[e] *= qscale;
                h[e] = __float2half_rn(x[e]);
                l[e] = __float2half_rn(x[e] - __half2float(h[e]));
            }
            frag(0, i) = make_uint2(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]));
            frag(1, i) = make_uint2(pack_h2(l[0], l[1]), pack_h2(l[2], l[3]));
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            const uint2 v = frag(0, ks * 32 + lane);
            qh[ks][0] = v.x;
            qh[ks][1] = v.y;
            if constexpr (QSPLIT) {
                const uint2 u = frag(1, ks * 32 + lane);
                ql[ks][0] = u.x;
                ql[ks][1] = u.y;
            }
        }
    }
    if constexpr (PRECISE) {
        // Short contexts: the table's f16 centroids (good to 1e-4) are not averaged out over enough positions, so
        // what their rounding left over goes into the upper halves of the table slots (free again now that every
        // warp has its q fragments) and every product gets a second term.
        __syncthreads();
        constexpr int kIdxMask = (1 << BITS) - 1;
        const float c_lo = a.book[lane & kIdxMask] * lut_alpha;
        for (int e = warp; e < 256; e += kMW) {
            const float lo = __shfl_sync(0xffffffffu, c_lo, e & kIdxMask), hi = __shfl_sync(0xffffffffu, c_lo, (e >> 4) & kIdxMask);
            const float2 hf = __half22float2(__floats2half2_rn(lo, hi));
            *reinterpret_cast<__half2 *>(lut_ptr + e * 256 + 128 + lane * 4) = __floats2half2_rn(lo - hf.x, hi - hf.y);
        }
        __syncthreads();
    }
    BK_STAMP(2);
    // ---- fused append: warps 0 and 1 of the CTA that scans the last chunk of this kv head store the
    // head's new K and V rows, exactly as the append kernel would (src/forward.rs:259-285; the rope
    // row of the new token is the q position's).  Only the chunk's last tile sees those rows; it is
    // issued by warp 0 after both rows are stored and fenced.
    bool inject = false;
    if (appender && warp < 2) {
        const float *src = (warp == 0 ? a.new_k : a.new_v) + ((size_t)meta.slot[s] * a.n_kv + kv) * kHd;
        float *sx = o.new_row[warp];
        const float *book = o.book[warp];
        reinterpret_cast<float4 *>(sx)[lane] = reinterpret_cast<const float4 *>(src)[lane];
        reinterpret_cast<float4 *>(sx)[lane + 32] = reinterpret_cast<const float4 *>(src)[lane + 32];
        __syncwarp();
        if (warp == 0 && a.k_norm_w) {  // per-head RMSNorm of the new k row, bit-exact (src/forward.rs:244-245)
            float sc = 0.f;
            if (lane == 0) sc = rms_scale_ref(sx, kHd, a.eps);
            sc = __shfl_sync(0xffffffffu, sc, 0);
            for (int i = lane; i < kHd; i += 32) sx[i] = __fmul_rn(__fmul_rn(sx[i], sc), a.k_norm_w[i]);
            __syncwarp();
        }
        if (warp == 0 && !a.no_rope) {
            const int half = a.n_rot >> 1;
            for (int j = lane; j < half; j += 32) {
                float x0 = sx[j], x1 = sx[j + half];
                rope_pair(x0, x1, o.rope_row[j]);
                sx[j] = x0;
                sx[j + half] = x1;
            }
            __syncwarp();
        }
        float n = 0.f;
        if (lane == 0) n = serial_norm(sx, kHd);
        n = __shfl_sync(0xffffffffu, n, 0);
        const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
        uint64_t packed = 0;
#pragma unroll
        for (int pr = 0; pr < 4; pr++) {
            const int i = lane * 4 + pr;  // pair index: coordinates 2i, 2i+1
            float r0, r1;
            givens_fwd(__fmul_rn(sx[2 * i], inv), __fmul_rn(sx[2 * i + 1], inv), o.givens[2 * i], o.givens[2 * i + 1], r0, r1);
            packed |= (uint64_t)nearest_centroid_fast<BITS>(r0, book) << (BITS * (2 * pr));
            packed |= (uint64_t)nearest_centroid_fast<BITS>(r1, book) << (BITS * (2 * pr + 1));
        }
        const size_t row = seq_rows + (size_t)(n_pos - 1) * a.n_kv + kv;
        store_group8<BITS>((warp == 0 ? a.k_rows_w : a.v_rows_w) + row * kRowBytes, lane, packed);
        if (lane == 0) (warp == 0 ? a.k_norms_w : a.v_norms_w)[row] = n;
        __threadfence();
        asm volatile("fence.proxy.async;\n" ::: "memory");  // generic-proxy stores before the TMA reads of the last tile
        __syncwarp();
        if (warp == 1) {
            asm volatile("bar.arrive 1, 64;\n" ::: "memory");
        } else {
            asm volatile("bar.sync 1, 64;\n" ::: "memory");      // the V row of warp 1 is stored too
            asm volatile("fence.proxy.async;\n" ::: "memory");
            inject = true;
        }
    }
    BK_STAMP(3);

    float acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    float M0 = -CUDART_INF_F, M1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    auto compute_tile = [&](int lt, uint32_t st_addr) {
        const int pb = (tile0 + lt) * kTile;
        // row block m (0, 1) holds positions pb + 16 m + {row_of(g), row_of(g) + 8}; their norms for this kv head
        float kn[2][2], vn[2][2];
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const uint32_t na = st_addr + 2 * kTileBytes + (uint32_t)(((16 * m + row_of<BITS>(g)) * a.n_kv + kv) * 4), step = (uint32_t)(8 * a.n_kv * 4);
            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(kn[m][0]) : "r"(na));
            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(kn[m][1]) : "r"(na + step));
            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(vn[m][0]) : "r"(na + norm_pad));
            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(vn[m][1]) : "r"(na + norm_pad + step));
        }
        // ---- scores^T = Kc . Q^T : per row block four independent accumulator chains ----------
        float S[2][4][4];
#pragma unroll
        for (int m = 0; m < 2; m++)
#pragma unroll
            for (int i = 0; i < 4; i++) S[m][i][0] = S[m][i][1] = S[m][i][2] = S[m][i][3] = 0.f;
        // 3 bit: coordinates 64 t .. 64 t + 63 of a row are 24 bytes, read once as three 8-byte words and
        // widened group by group to words of eight nibbles: [m][row g / g + 8][c][w]
        uint32_t k3[BITS != 4 ? 2 : 1][2][2][4];
        if constexpr (BITS == 2) {
            // 2 bit: coordinates 64 t .. 64 t + 63 of a row are one 16-byte chunk (swizzled), four words of sixteen indices
#pragma unroll
            for (int m = 0; m < 2; m++)
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint32_t row = (uint32_t)(16 * m + 8 * hh + row_of<BITS>(g));
                    const uint4 u = lds128(st_addr + row * kRowBytes + ((((uint32_t)t) ^ ((row >> 1) & 3u)) << 4));
                    k3[m][hh][0][0] = expand16(u.x);
                    k3[m][hh][0][1] = expand16(u.x >> 16);
                    k3[m][hh][0][2] = expand16(u.y);
                    k3[m][hh][0][3] = expand16(u.y >> 16);
                    k3[m][hh][1][0] = expand16(u.z);
                    k3[m][hh][1][1] = expand16(u.z >> 16);
                    k3[m][hh][1][2] = expand16(u.w);
                    k3[m][hh][1][3] = expand16(u.w >> 16);
                }
        }
        if constexpr (BITS == 3) {
#pragma unroll
            for (int m = 0; m < 2; m++)
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint32_t addr = st_addr + (uint32_t)((16 * m + 8 * hh + row_of<BITS>(g)) * kRowBytes) + 24 * t;
                    const uint2 u01 = lds64(addr), u23 = lds64(addr + 8), u45 = lds64(addr + 16);
                    k3[m][hh][0][0] = expand24(u01.x);
                    k3[m][hh][0][1] = expand24(__funnelshift_r(u01.x, u01.y, 24));
                    k3[m][hh][0][2] = expand24(__funnelshift_r(u01.y, u23.x, 16));
                    k3[m][hh][0][3] = expand24(u23.x >> 8);
                    k3[m][hh][1][0] = expand24(u23.y);
                    k3[m][hh][1][1] = expand24(__funnelshift_r(u23.y, u45.x, 24));
                    k3[m][hh][1][2] = expand24(__funnelshift_r(u45.x, u45.y, 16));
                    k3[m][hh][1][3] = expand24(u45.y >> 8);
                }
        }
#pragma unroll
        for (int c = 0; c < 2; c++) {
            // coordinates 64 t + 32 c .. + 31 of rows g and g + 8 of both row blocks, four words of eight nibbles each
            uint32_t kg[2][4], kh[2][4];
#pragma unroll
            for (int m = 0; m < 2; m++) {
                [[maybe_unused]] const uint32_t k_row = st_addr + (uint32_t)((16 * m + row_of<BITS>(g)) * kRowBytes);
                if constexpr (BITS == 4) {
                    // swizzled: the 16-byte chunk index is XORed with (row & 7); rows g, g + 8, g + 16, g + 24 share it
                    const uint32_t koff = (uint32_t)(((2 * t + c) ^ g) << 4);
                    const uint4 rk_g = lds128(k_row + koff), rk_h = lds128(k_row + 8 * kRowBytes + koff);
                    kg[m][0] = rk_g.x; kg[m][1] = rk_g.y; kg[m][2] = rk_g.z; kg[m][3] = rk_g.w;
                    kh[m][0] = rk_h.x; kh[m][1] = rk_h.y; kh[m][2] = rk_h.z; kh[m][3] = rk_h.w;
                } else {
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        kg[m][w] = k3[m][0][c][w];
                        kh[m][w] = k3[m][1][c][w];
                    }
                }
            }
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const int ks = c * 8 + w * 2;
#pragma unroll
                for (int m = 0; m < 2; m++) {
                    if constexpr (PRECISE) {  // centroid = table value + remainder: a third term per fragment
                        uint32_t a0, a1, a2, a3, r0, r1, r2, r3;
                        lut2<0>(kg[m][w], lane_base, a0, r0);
                        lut2<0>(kh[m][w], lane_base, a1, r1);
                        lut2<1>(kg[m][w], lane_base, a2, r2);
                        lut2<1>(kh[m][w], lane_base, a3, r3);
                        mma16816(S[m][c], a0, a1, a2, a3, qh[ks][0], qh[ks][1]);
                        mma16816(S[m][2 + c], r0, r1, r2, r3, qh[ks][0], qh[ks][1]);
                        if constexpr (QSPLIT) mma16816(S[m][2 + c], a0, a1, a2, a3, ql[ks][0], ql[ks][1]);
                        lut2<2>(kg[m][w], lane_base, a0, r0);
                        lut2<2>(kh[m][w], lane_base, a1, r1);
                        lut2<3>(kg[m][w], lane_base, a2, r2);
                        lut2<3>(kh[m][w], lane_base, a3, r3);
                        mma16816(S[m][2 + c], a0, a1, a2, a3, qh[ks + 1][0], qh[ks + 1][1]);
                        mma16816(S[m][c], r0, r1, r2, r3, qh[ks + 1][0], qh[ks + 1][1]);
                        if constexpr (QSPLIT) mma16816(S[m][c], a0, a1, a2, a3, ql[ks + 1][0], ql[ks + 1][1]);
                    } else {
                    {
                        const uint32_t a0 = lut<0>(kg[m][w], lane_base), a1 = lut<0>(kh[m][w], lane_base);
                        const uint32_t a2 = lut<1>(kg[m][w], lane_base), a3 = lut<1>(kh[m][w], lane_base);
                        mma16816(S[m][c], a0, a1, a2, a3, qh[ks][0], qh[ks][1]);
                        if constexpr (QSPLIT) mma16816(S[m][2 + c], a0, a1, a2, a3, ql[ks][0], ql[ks][1]);
                    }
                    {
                        const uint32_t a0 = lut<2>(kg[m][w], lane_base), a1 = lut<2>(kh[m][w], lane_base);
                        const uint32_t a2 = lut<3>(kg[m][w], lane_base), a3 = lut<3>(kh[m][w], lane_base);
                        mma16816(S[m][2 + c], a0, a1, a2, a3, qh[ks + 1][0], qh[ks + 1][1]);
                        if constexpr (QSPLIT) mma16816(S[m][c], a0, a1, a2, a3, ql[ks + 1][0], ql[ks + 1][1]);
                    }
                    }
                }
            }
        }
        // ---- online softmax in the exp2 domain; reference point = max of s + log2||v|| -------
        float tt[2][4], sv[2][4];
        bool ok[2][2];
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
        for (int m = 0; m < 2; m++) {
            ok[m][0] = pb + 16 * m + row_of<BITS>(g) < n_pos;
            ok[m][1] = pb + 16 * m + row_of<BITS>(g) + 8 < n_pos;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = i >> 1;  // accumulator entries 0, 1: row g; 2, 3: row g + 8; even: head 2t, odd: head 2t + 1
                const float sc = (S[m][0][i] + S[m][1][i]) + (S[m][2][i] + S[m][3][i]);
                sv[m][i] = sc * kn[m][r];
                tt[m][i] = ok[m][r] ? sv[m][i] + fast_log2(fmaxf(vn[m][r], 1e-30f)) : -CUDART_INF_F;
            }
            mx0 = fmaxf(mx0, fmaxf(tt[m][0], tt[m][2]));
            mx1 = fmaxf(mx1, fmaxf(tt[m][1], tt[m][3]));
        }
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const bool grow = (mx0 > M0) || (mx1 > M1);
        if (__any_sync(0xffffffffu, grow)) {
            const float n0 = fmaxf(M0, mx0), n1 = fmaxf(M1, mx1);
            const float c0 = fast_exp2(M0 - n0), c1 = fast_exp2(M1 - n1);  // 0 on the first tile
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
        uint32_t b0[2], b1[2];
        [[maybe_unused]] uint32_t b0l[2] = {0u, 0u}, b1l[2] = {0u, 0u};  // PRECISE: what the weights' rounding to f16 left over
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const float w00 = fast_exp2(tt[m][0] - M0) * kWScale, w01 = fast_exp2(tt[m][1] - M1) * kWScale;
            const float w10 = fast_exp2(tt[m][2] - M0) * kWScale, w11 = fast_exp2(tt[m][3] - M1) * kWScale;
            l0 += (ok[m][0] ? fast_exp2(sv[m][0] - M0) : 0.f) + (ok[m][1] ? fast_exp2(sv[m][2] - M0) : 0.f);
            l1 += (ok[m][0] ? fast_exp2(sv[m][1] - M1) : 0.f) + (ok[m][1] ? fast_exp2(sv[m][3] - M1) : 0.f);
            const __half2 pl = __floats2half2_rn(w00, w01), ph = __floats2half2_rn(w10, w11);
            b0[m] = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&pl));  // head g; pos 2t, 2t+1
            b1[m] = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph));  // head g; pos 2t+8, 2t+9
            if constexpr (PRECISE) {
                const float2 fl = __half22float2(pl), fh = __half22float2(ph);
                const __half2 ql2 = __floats2half2_rn(w00 - fl.x, w01 - fl.y), qh2 = __floats2half2_rn(w10 - fh.x, w11 - fh.y);
                b0l[m] = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ql2));
                b1l[m] = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&qh2));
            }
        }
        // ---- out^T += Vc^T . W : MMA j covers coordinates 32g + 2j (rows g) and 32g + 2j + 1 (rows g+8)
        const uint32_t v_tile = st_addr + kTileBytes;
        const uint32_t r0 = (uint32_t)row_of<BITS>(2 * t), r1 = (uint32_t)row_of<BITS>(2 * t + 1);
#pragma unroll
        for (int m = 0; m < 2; m++) {
            // coordinates 32 g .. 32 g + 31 of position rows 2t, 2t+1, 2t+8, 2t+9 of this row block, four words each
            const uint32_t v_blk = v_tile + (uint32_t)(16 * m * kRowBytes);
            const uint32_t bm0 = m ? b0[1] : b0[0], bm1 = m ? b1[1] : b1[0];
            [[maybe_unused]] const uint32_t bm0l = m ? b0l[1] : b0l[0], bm1l = m ? b1l[1] : b1l[0];
            uint32_t x0[4], x1[4], x2[4], x3[4];
            if constexpr (BITS == 4) {  // chunk g of each row; rows r and r + 8 share the swizzle
                const uint32_t vo0 = r0 * kRowBytes + (((uint32_t)g ^ (r0 & 7)) << 4), vo1 = r1 * kRowBytes + (((uint32_t)g ^ (r1 & 7)) << 4);
                const uint4 rv0 = lds128(v_blk + vo0), rv1 = lds128(v_blk + vo1);
                const uint4 rv2 = lds128(v_blk + 8 * kRowBytes + vo0), rv3 = lds128(v_blk + 8 * kRowBytes + vo1);
                x0[0] = rv0.x; x0[1] = rv0.y; x0[2] = rv0.z; x0[3] = rv0.w;
                x1[0] = rv1.x; x1[1] = rv1.y; x1[2] = rv1.z; x1[3] = rv1.w;
                x2[0] = rv2.x; x2[1] = rv2.y; x2[2] = rv2.z; x2[3] = rv2.w;
                x3[0] = rv3.x; x3[1] = rv3.y; x3[2] = rv3.z; x3[3] = rv3.w;
            } else if constexpr (BITS == 2) {  // 8 bytes per row (chunk g / 2, swizzled, half g & 1), widened
                auto load_v = [&](uint32_t row, uint32_t (&out)[4]) {
                    const uint2 u = lds64(v_blk + row * kRowBytes + (((uint32_t)(g >> 1) ^ ((row >> 1) & 3u)) << 4) + (uint32_t)((g & 1) * 8));
                    out[0] = expand16(u.x);
                    out[1] = expand16(u.x >> 16);
                    out[2] = expand16(u.y);
                    out[3] = expand16(u.y >> 16);
                };
                load_v(r0, x0);
                load_v(r1, x1);
                load_v(r0 + 8, x2);
                load_v(r1 + 8, x3);
            } else {  // 12 bytes per row: three 4-byte reads, widened
                auto load_v = [&](uint32_t addr, uint32_t (&out)[4]) {
                    const uint32_t u0 = lds32(addr), u1 = lds32(addr + 4), u2 = lds32(addr + 8);
                    out[0] = expand24(u0);
                    out[1] = expand24(__funnelshift_r(u0, u1, 24));
                    out[2] = expand24(__funnelshift_r(u1, u2, 16));
                    out[3] = expand24(u2 >> 8);
                };
                load_v(v_blk + r0 * kRowBytes + 12 * g, x0);
                load_v(v_blk + r1 * kRowBytes + 12 * g, x1);
                load_v(v_blk + (r0 + 8) * kRowBytes + 12 * g, x2);
                load_v(v_blk + (r1 + 8) * kRowBytes + 12 * g, x3);
            }
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const uint32_t msk = 0x0f0f0f0fu;
                const uint32_t lo01 = (x0[w] & msk) | ((x1[w] & msk) << 4), hi01 = ((x0[w] >> 4) & msk) | (x1[w] & ~msk);
                const uint32_t lo23 = (x2[w] & msk) | ((x3[w] & msk) << 4), hi23 = ((x2[w] >> 4) & msk) | (x3[w] & ~msk);
                if constexpr (PRECISE) {
                    auto both = [&]<int B>(float (&dst)[4]) {
                        uint32_t a0, a1, a2, a3, r0, r1, r2, r3;
                        lut2<B>(lo01, lane_base, a0, r0);
                        lut2<B>(hi01, lane_base, a1, r1);
                        lut2<B>(lo23, lane_base, a2, r2);
                        lut2<B>(hi23, lane_base, a3, r3);
                        mma16816(dst, a0, a1, a2, a3, bm0, bm1);
                        mma16816(dst, r0, r1, r2, r3, bm0, bm1);
                        mma16816(dst, a0, a1, a2, a3, bm0l, bm1l);
                    };
                    both.template operator()<0>(acc[4 * w + 0]);
                    both.template operator()<1>(acc[4 * w + 1]);
                    both.template operator()<2>(acc[4 * w + 2]);
                    both.template operator()<3>(acc[4 * w + 3]);
                } else {
                mma16816(acc[4 * w + 0], lut<0>(lo01, lane_base), lut<0>(hi01, lane_base), lut<0>(lo23, lane_base),
                         lut<0>(hi23, lane_base), bm0, bm1);
                mma16816(acc[4 * w + 1], lut<1>(lo01, lane_base), lut<1>(hi01, lane_base), lut<1>(lo23, lane_base),
                         lut<1>(hi23, lane_base), bm0, bm1);
                mma16816(acc[4 * w + 2], lut<2>(lo01, lane_base), lut<2>(hi01, lane_base), lut<2>(lo23, lane_base),
                         lut<2>(hi23, lane_base), bm0, bm1);
                mma16816(acc[4 * w + 3], lut<3>(lo01, lane_base), lut<3>(hi01, lane_base), lut<3>(lo23, lane_base),
                         lut<3>(hi23, lane_base), bm0, bm1);
                }
            }
        }
    };

    // ---- scan: the stages are used round robin; a freed stage takes the tile drawn one step earlier
    {
        if (inject && in_stage[0] < 0) {  // a chunk so short that warp 0 holds nothing yet
            in_stage[0] = n_tiles - 1;
            issue_tile(n_tiles - 1, 0);
            inject = false;
        }
        const uint32_t ctr_addr = other_addr + (uint32_t)offsetof(Other, next_tile);
        int drawn = 0;
        auto draw = [&]() {
            if (lane == 0) asm volatile("atom.shared.add.u32 %0, [%1], 1;\n" : "=r"(drawn) : "r"(ctr_addr) : "memory");
        };
        if (dyn) draw();
        auto held = [&](int i) -> int {
            int r = in_stage[0];
#pragma unroll
            for (int j = 1; j < kMaxStages; j++) r = (i == j) ? in_stage[j] : r;
            return r;
        };
        int n_held = 0;
#pragma unroll
        for (int j = 0; j < kMaxStages; j++) n_held += in_stage[j] >= 0 ? 1 : 0;
        int st = 0;
        uint32_t phase = 0;  // bit st: the parity the next wait on stage st looks for
        while (n_held > 0) {
            const int lt = held(st);
            if (lt >= 0) {
                wait_tile(st, (phase >> st) & 1u);
                phase ^= 1u << st;
#ifdef BK_PHASE
                if (!(a.dyn & 2))  // tuning builds: dyn bit 1 = stream the tiles without computing on them
#endif
                compute_tile(lt, stage_of(st));
                __syncwarp();  // every lane has read the stage: lane 0 may refill it
                int nu;
                if (inject) {  // warp 0 of the appending CTA: the rows are stored, take their tile now
                    nu = n_tiles - 1;
                    inject = false;
                } else if (dyn) {
                    nu = __shfl_sync(0xffffffffu, drawn, 0);
                    if (nu < n_pool) draw();  // the draw after this one
                    else nu = -1;
                } else {
                    nu = fixed_tile(i_next++);
                    if (nu >= n_pool) nu = -1;
                }
                if (nu >= 0) issue_tile(nu, st);
                else n_held--;
#pragma unroll
                for (int j = 0; j < kMaxStages; j++) in_stage[j] = (st == j) ? nu : in_stage[j];
            }
            if (++st == n_stages) st = 0;
        }
    }
    BK_STAMP(4);

    // The scan is over: a dependent kernel (launched with programmatic serialization) may start
    // its own constant-table set-up on the SMs this kernel frees while its last CTAs merge.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

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
    static_assert((size_t)kMW * 6 * kHeadStride * sizeof(float) <= kLutBytes, "merge area does not fit the table");
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
            sums[r] = 0.f;
#pragma unroll
            for (int w = 0; w < kMW; w++) sums[r] += area[((size_t)w * NREP + r) * kHeadStride + idx];
        }
    }
    __syncthreads();
    float *s_acc = area;  // [NREP][256]
#pragma unroll
    for (int r = 0; r < NREP; r++) s_acc[r * kHd + tid] = sums[r];
    __syncthreads();

    // Free shared memory for the combine: from behind the merged accumulator (which sits at the
    // start of the table) to the bookkeeping block, i.e. the rest of the table and the ring behind it.
    FinishSmem fs;
    fs.addr = lut_addr + (uint32_t)(NREP * kHd * sizeof(float));
    fs.bytes = other_addr - fs.addr;
    fs.bar = other_addr + (uint32_t)offsetof(Other, fin_bar);
    fs.ptr = smem_raw + (fs.addr - base);
    fs.err_flag = err_flag;
    BK_STAMP(5);
    const int first_item = meta.item_start[s] + kv * n_chunks;
    finish_item<NREP, true>(a, meta.slot[s], s, kv, item, n_chunks, first_item, s_acc, o.M, o.L, &o.last, true, o.givens, fs);
    BK_STAMP(9);
}

template <int BITS, int NREP, bool QSPLIT, bool PRECISE = false>
bk_status launch_one(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float alpha) {
    auto *kernel = decode_p4_mma_kernel<BITS, NREP, QSPLIT, PRECISE>;
    // Dynamic shared memory: everything the SM allows beyond the kernel's static part.  The kernel
    // lays out table, bookkeeping and as many ring stages as fit.
    static std::atomic<size_t> smem_for[64] = {};  // per device; racing first calls compute the same value
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, BK_ERR_UNSUPPORTED, "decode (mma): device index above 63");
    if (smem_for[dev].load() == 0) {
        cudaFuncAttributes fa;
        BK_CUDA(ctx, cudaFuncGetAttributes(&fa, kernel));
        int optin = 0;
        BK_CUDA(ctx, cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        const size_t dyn = (size_t)optin - fa.sharedSizeBytes;
        const size_t stage = 2 * (size_t)Width<BITS>::kTileBytes + 2 * 1024;
        const size_t need = 2 * (size_t)kLutBytes + kOtherBytes + (size_t)kMW * stage;  // the table may need up to 64 KiB of alignment
        if (dyn < need) return fail(ctx, BK_ERR_UNSUPPORTED, "decode (mma): not enough shared memory per block on this device");
        BK_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
        smem_for[dev].store(dyn);
    }
    const size_t smem = smem_for[dev].load();
    if (!a.h_tmap_k || !a.h_tmap_v) return fail(ctx, BK_ERR_INVALID, "decode (mma): the cache has no tensor maps");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)m.n_items);
    cfg.blockDim = dim3(kMT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol.* in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BK_CUDA(ctx, cudaLaunchKernelEx(&cfg, kernel, a, m, alpha, (uint32_t)smem, ctx->d_err,
                                    *static_cast<const CUtensorMap *>(a.h_tmap_k),
                                    *static_cast<const CUtensorMap *>(a.h_tmap_v)));
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace

// Tensor maps over the K and V rows of a cache whose rows are k_row_bytes / v_row_bytes long (128 for
// 4-bit planar, 96 for 3-bit, 512 for f16, 1024 for f32): dims (row_bytes, n_kv, positions of all layers and sequences), box
// (128 bytes or the whole row, 1, box_rows positions), 128-byte swizzle where rows allow it.
// Built once per cache.
bk_status make_tile_tensor_maps(bk_ctx *ctx, const void *k_rows, const void *v_rows, size_t k_row_bytes, size_t v_row_bytes, int n_kv,
                                size_t total_pos, int box_rows, void *out_k, void *out_v) {
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::atomic<EncodeFn> encode_fn{nullptr};
    EncodeFn encode = encode_fn.load();
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        BK_CUDA(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
        if (!fn || qr != cudaDriverEntryPointSuccess)
            return fail(ctx, BK_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available in this driver");
        encode = (EncodeFn)fn;
        encode_fn.store(encode);
    }
    if (total_pos >= (size_t)1 << 31) return fail(ctx, BK_ERR_UNSUPPORTED, "cache has more than 2^31 positions");
    const void *ptrs[2] = {k_rows, v_rows};
    const size_t row_bytes_of[2] = {k_row_bytes, v_row_bytes};
    void *outs[2] = {out_k, out_v};
    for (int i = 0; i < 2; i++) {
        const size_t row_bytes = row_bytes_of[i];
        // rows of a multiple of 128 bytes travel as 128-byte swizzled slabs; 64-byte rows (2 bit) whole, with the
        // 64-byte swizzle; other short rows (96 bytes: 3 bit) as whole dense rows without a swizzle
        const bool swizzled = row_bytes % 128 == 0, swizzled64 = row_bytes == 64;
        if (!swizzled && (row_bytes % 16 != 0 || row_bytes > 256))
            return fail(ctx, BK_ERR_UNSUPPORTED, "tensor maps need rows of a multiple of 16 bytes");
        const cuuint64_t dims[3] = {(cuuint64_t)row_bytes, (cuuint64_t)n_kv, (cuuint64_t)total_pos};
        const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)row_bytes * n_kv};
        const cuuint32_t box[3] = {swizzled ? 128u : (cuuint32_t)row_bytes, 1, (cuuint32_t)box_rows};
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = encode(static_cast<CUtensorMap *>(outs[i]), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                                  const_cast<void *>(ptrs[i]), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : swizzled64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(ctx, BK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    }
    return BK_OK;
}

bool decode_p4_mma_supported(const DecodeArgs &a) {
    const int n_rep = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    // the norms of a tile travel as a 16-byte aligned bulk copy: n_ctx * n_kv must be a multiple of 4;
    // the in-lane rope needs both coordinates of a pair in one lane (n_rot = 64) or exactly 1 or 2 lanes apart
    const bool rope_ok = a.no_rope || a.n_rot == 0 || a.n_rot == 64 || a.n_rot == 128 || a.n_rot == 256;
    return a.h_tmap_k && a.h_tmap_v && (a.seq_stride_rows % 4 == 0) && a.k_kind == ROW_PLANAR && a.v_kind == ROW_PLANAR && (a.bits == 4 || a.bits == 3 || a.bits == 2) &&
           a.n_kv <= 8 && rope_ok && (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 6);
}

bk_status launch_decode_p4_mma(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float alpha, bool qsplit, bool precise) {
    if (m.n_items <= 0) return BK_OK;
    const int n_rep = a.n_head / a.n_kv;
    // (the precise form always carries the q split as well: it exists for accuracy)
#define BK_MMA_BITS(B, R)                                                        \
    if (a.bits == B) {                                                           \
        if (precise) return launch_one<B, R, true, true>(ctx, a, m, alpha);      \
        return qsplit ? launch_one<B, R, true>(ctx, a, m, alpha) : launch_one<B, R, false>(ctx, a, m, alpha); \
    }
#define BK_MMA_CASE(R) \
    case R:            \
        BK_MMA_BITS(3, R) BK_MMA_BITS(2, R) BK_MMA_BITS(4, R) break;
    switch (n_rep) {
        BK_MMA_CASE(1)
        BK_MMA_CASE(2)
        BK_MMA_CASE(4)
        BK_MMA_CASE(6)
        default: return fail(ctx, BK_ERR_UNSUPPORTED, "decode (mma): n_head/n_kv must be 1, 2, 4 or 6");
    }
#undef BK_MMA_CASE
#undef BK_MMA_BITS
    return fail(ctx, BK_ERR_UNSUPPORTED, "decode (mma): index width must be 4, 3 or 2");
}

}  // namespace bk

#ifdef BK_PHASE
// Tuning builds only: copy the per-CTA time stamps out (and clear them).
extern "C" __attribute__((visibility("default"))) int bk_debug_phase(unsigned long long *out, int clear) {
    if (out && cudaMemcpyFromSymbol(out, bk::g_phase, sizeof(bk::g_phase)) != cudaSuccess) return 1;
    if (clear) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, bk::g_phase) != cudaSuccess || cudaMemset(p, 0, sizeof(bk::g_phase)) != cudaSuccess) return 2;
    }
    return 0;
}
#endif
