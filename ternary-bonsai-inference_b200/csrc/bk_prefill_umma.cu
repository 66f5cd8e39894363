// Batched (prefill) attention over a 4-, 3- or 2-bit planar cache, or an f16 or f32 cache, on the
// 5th-generation tensor cores: the same work split, operands and arithmetic as bk_prefill.cu
// (which documents them and stays as the mma.sync form), with both contractions issued as
// tcgen05.mma and the accumulators in tensor memory.
//
// One CTA = 128 query rows (M = 128) of one kv head over one context chunk; 8 warps.  Per tile
// of 32 positions:
//   1. all warps dequantize the packed K rows once into shared memory as f16 (for 4 bit also the
//      rounding remainders, as rows 32-63 of the same K-major, 128-byte-swizzled operand tile);
//   2. one thread issues S[128 x 32] = Q . K^T as 16 K-steps x (q_hi [k_hi; k_lo] with N = 64, then
//      q_lo k_hi with N = 32) into tensor-memory columns and commits to an mbarrier; while those
//      MMAs run, all warps dequantize V (hi and lo tiles, read later as the MN-major B operand);
//   3. warps 0-3 (thread = query row: tensor-memory lane r is row r) read their row of S with
//      tcgen05.ld, scale by ||k||, apply the causal limit, update the running reference R of
//      s + log2 ||v|| LAZILY (only when the row maximum exceeds R by more than 8: the weights
//      p = 2^(t - R) * 64 then stay below 2^14 in f16), rescale their row of O in tensor memory when
//      R moved, and write the weights as f16 hi + lo into the no-swizzle K-major P tiles;
//   4. the same thread issues O[128 x 256] += P . V as 2 K-steps x (p_hi v_hi + p_lo v_hi + p_hi v_lo)
//      into 256 tensor-memory columns and commits.
// f16 caches (BITS = 16) skip the dequantization: the TMA engine drops their rows, which are the
// operands as stored, into two shared-memory stages through the cache's swizzled tensor maps.
// f32 caches (BITS = 32) take the place of the dequantization with a split of every float into f16 hi + lo
// (both K parts side by side as for 4 bit, both V parts as for 4 bit).
// For packed and f32 caches the K rows of tile t + 1 are dequantized right after the O products of tile t are
// issued (the K tile is free once S of tile t is complete), so that step runs under the tensor cores' work.
// Every mbarrier wait is bounded (a time-out raises the context's error flag and the kernel runs
// on to its end, where the tensor memory is always released).  The packed rows of the next tile
// are fetched into registers (f16: into the other stage) while the current one is computed.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <atomic>

#include "bk_device.cuh"
#include "bk_internal.h"
#include "bk_mma_common.cuh"
#include "bk_umma.cuh"

namespace bk {

namespace {

constexpr int kUW = 8, kUT = kUW * 32;
constexpr int kRows = 128;  // query rows per CTA = tensor-memory lanes
constexpr int kTK = 32;     // positions per tile
constexpr float kPScale = 64.0f;
constexpr float kLazy = 8.0f;  // the reference moves when a row maximum exceeds it by more than this (log2 units)

constexpr uint32_t kQSlab = kRows * 128, kQTile = 4 * kQSlab;  // 16 KiB per 64-coordinate slab, 64 KiB per tile
constexpr uint32_t kKVSlab = kTK * 128, kKVTile = 4 * kKVSlab;  // 4 KiB, 16 KiB
constexpr uint32_t kPChunk = (kRows / 8) * 128, kPTile = 4 * kPChunk;  // 2 KiB per 8 positions, 8 KiB
// offsets from the 1024-byte aligned base
constexpr uint32_t oQhi = 0, oQlo = kQTile, oKhi = 2 * kQTile, oKlo = oKhi + kKVTile, oVhi = oKlo + kKVTile,
                   oVlo = oVhi + kKVTile, oPhi = oVlo + kKVTile, oPlo = oPhi + kPTile, oSmall = oPlo + kPTile;
struct SmallU {
    float kn[kTK], lv[kTK];  // ||k|| and log2 ||v|| of the tile's positions
    float givens[kHd];
    __half table[16], table_lo[16];
    unsigned long long bar_s, bar_o;
    unsigned long long bar_t[2];  // f16 caches: the TMA engine fills two K/V stages
    uint32_t tmem_slot;
};
constexpr uint32_t kUmmaSmem = oSmall + sizeof(SmallU) + 1024;  // + alignment slack
constexpr uint32_t kTmemCols = 512, kColS = 0, kColO = 64;  // S: 32 (+32 for the k_lo term) columns, O: 256

__device__ __forceinline__ uint32_t sw_off(int rows, int row, int chunk) {  // as tile_off in bk_prefill.cu
    return (uint32_t)((chunk >> 3) * rows * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
__device__ __forceinline__ uint32_t expand24u(uint32_t y) {
    y &= 0x00ffffffu;
    y += (y & 0x00fff000u) * 15u;
    y += (y & 0x0fc00fc0u) * 3u;
    y += (y & 0x38383838u);
    return y;
}
__device__ __forceinline__ uint32_t expand16u(uint32_t y) {  // eight 2-bit indices -> eight nibbles
    y &= 0x0000ffffu;
    y = (y | (y << 8)) & 0x00ff00ffu;
    y = (y | (y << 4)) & 0x0f0f0f0fu;
    y = (y | (y << 2)) & 0x33333333u;
    return y;
}
// 32 coordinates (four words of eight nibbles) -> 32 halfs as four 16-byte chunks of a tile row.
// The table sits in registers: lane i holds (hi | lo << 16) of centroid i & 15, one shuffle looks
// both parts of an index up, and no shared-memory bank is involved.
template <bool LO>
__device__ __forceinline__ void dequant_store_shfl(const uint32_t (&w)[4], uint32_t tab, uint8_t *tile_hi, uint8_t *tile_lo, int rows,
                                                   int row_hi, int row_lo, int chunk0) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const uint32_t v0 = __shfl_sync(0xffffffffu, tab, (w[j] >> (8 * e)) & 15u);
            const uint32_t v1 = __shfl_sync(0xffffffffu, tab, (w[j] >> (8 * e + 4)) & 15u);
            h[e] = __byte_perm(v0, v1, 0x5410);
            l[e] = __byte_perm(v0, v1, 0x7632);
        }
        *reinterpret_cast<uint4 *>(tile_hi + sw_off(rows, row_hi, chunk0 + j)) = make_uint4(h[0], h[1], h[2], h[3]);
        if (LO) *reinterpret_cast<uint4 *>(tile_lo + sw_off(rows, row_lo, chunk0 + j)) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

struct PrefillUArgs {
    DecodeArgs d;
    int seq, pos0, n_tokens, tq, n_blocks, n_chunks;
    float lut_alpha;
    float *scratch;
    int *err_flag;
};

template <int BITS, int NREP, bool VF32 = false>
__global__ void __launch_bounds__(kUT, 1)
prefill_umma_kernel(PrefillUArgs pa, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const DecodeArgs &a = pa.d;
    const uint32_t base0 = (uint32_t)__cvta_generic_to_shared(smem_raw), base = (base0 + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - base0);
    SmallU &ss = *reinterpret_cast<SmallU *>(sm + oSmall);
    const uint32_t bar_s = base + oSmall + (uint32_t)offsetof(SmallU, bar_s), bar_o = base + oSmall + (uint32_t)offsetof(SmallU, bar_o);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // BITS = 16 stands for an f16 cache: its rows ARE the operands, so the TMA engine drops them into
    // two shared-memory stages in the swizzled layout and nothing is dequantized (no table, no norms,
    // no Givens rotation); everything else is the same kernel.
    constexpr bool kF16 = BITS == 16;
    // BITS = 32 stands for an f32 cache: its rows are split into f16 hi + lo on their way into the operand tiles
    // (the lo tiles are the ones the 4-bit rows use for their rounding remainders); like f16 rows they are
    // neither rotated nor normalised.
    constexpr bool kF32 = BITS == 32, kRaw = kF16 || kF32;
    // VF32: the reference's K-only mode, planar K rows (BITS = 4 or 3) beside f32 V rows: the K side of the planar
    // kernel, the V side of the f32 one; q is rotated into the K rows' basis, the output is not rotated back.
    static_assert(!VF32 || BITS == 4 || BITS == 3, "VF32 goes with 4- or 3-bit K rows");
    constexpr bool kVRows32 = kF32 || VF32;   // V rows are floats
    constexpr bool kVPlanar = !kRaw && !VF32; // V rows are planar: a norm per row, the output is rotated back
    constexpr int kRowBytes = kF16 ? 512 : kF32 ? 1024 : 32 * BITS;  // (K rows; f32 V rows are 1024 bytes)
    // lo tiles: the rounding remainders of the 4-bit table (see bk_prefill.cu: it is only good to 1e-4), the lo parts
    // of f32 rows; beside raw V rows (several times larger than dequantized ones) the 3-bit table carries them too
    constexpr bool kLoTiles = BITS == 4 || kF32 || VF32;
    // The K operand holds k_hi in rows 0-31 of every slab and, for 4 bit, k_lo in rows 32-63: one MMA
    // with N = 64 then yields q_hi k_hi and q_hi k_lo side by side (q is re-read from shared memory
    // once instead of twice, and that read is what an N = 32 MMA waits for).
    constexpr int kKRows = kLoTiles ? 64 : 32;
    constexpr uint32_t kKSlab = kKRows * 128;

    // ---- which item (as in the mma.sync kernel) ---------------------------------------------
    const int item = blockIdx.x;
    // the blocks late in the prompt see the most rows: they go first
    const int chunk = item % pa.n_chunks, kv = (item / pa.n_chunks) % a.n_kv, blk = pa.n_blocks - 1 - item / (pa.n_chunks * a.n_kv);
    const int tok0 = blk * pa.tq, n_tok = min(pa.tq, pa.n_tokens - tok0), n_rows = n_tok * NREP;
    const int vis = pa.pos0 + tok0 + n_tok;
    const int L = ((vis + pa.n_chunks - 1) / pa.n_chunks + kTK - 1) / kTK * kTK;
    const int c0 = chunk * L, c1 = min(c0 + L, vis);
    const int n_tiles = c1 > c0 ? (c1 - c0 + kTK - 1) / kTK : 0;

    // ---- tables, barriers, tensor memory ----------------------------------------------------
    for (int i = tid; i < kHd; i += kUT) ss.givens[i] = a.givens[i];
    if (tid < 16) {
        const float c = kRaw ? 0.f : a.book[tid & ((1 << (kRaw ? 4 : BITS)) - 1)] * pa.lut_alpha;
        const __half h = __float2half_rn(c);
        ss.table[tid] = h;
        ss.table_lo[tid] = __float2half_rn(c - __half2float(h));
    }
    if (kRaw && tid < kTK) {  // no norms: ||k|| = 1, log2 ||v|| = 0
        ss.kn[tid] = 1.f;
        ss.lv[tid] = 0.f;
    }
    const uint32_t bar_t = base + oSmall + (uint32_t)offsetof(SmallU, bar_t);
    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_init(bar_t, 1);
        mbar_init(bar_t + 8, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (warp == 0) tmem_alloc(base + oSmall + (uint32_t)offsetof(SmallU, tmem_slot), kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = ss.tmem_slot;
    const uint32_t my_tmem = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's 32 lanes

    // O starts at zero (it is rescaled before the first product is added)
    if (warp < 4) {
        uint32_t z[32];
#pragma unroll
        for (int j = 0; j < 32; j++) z[j] = 0u;
        for (int b = 0; b < 8; b++) tmem_st32(my_tmem + kColO + 32 * b, z);
        tmem_wait_st();
    }

    // ---- q rows -> the two q tiles (rope, Givens, scale, f16 hi/lo); staged through the K tile ----
    {
        float *stage = reinterpret_cast<float *>(sm + oKhi) + warp * (kHd + 8);  // rows are padded by one float per 32 (see pad())
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
        for (int r = warp; r < kRows; r += kUW) {
            const bool real = r < n_rows;
            if (real) {
                float2 rc[4];
#pragma unroll
                for (int i = 0; i < 8; i++) stage[pad(lane + 32 * i)] = xn[i];
#pragma unroll
                for (int i = 0; i < 4; i++) rc[i] = rn[i];
                prefetch(r + kUW);
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
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                float o0 = 0.f, o1 = 0.f;
                if (real) {
                    const int d = 8 * lane + 2 * p;
                    if constexpr (kRaw) {
                        o0 = stage[pad(d)];
                        o1 = stage[pad(d + 1)];
                    } else {
                        givens_fwd(stage[pad(d)], stage[pad(d + 1)], ss.givens[d], ss.givens[d + 1], o0, o1);
                    }
                    o0 *= qscale;
                    o1 *= qscale;
                }
                const __half h0 = __float2half_rn(o0), h1 = __float2half_rn(o1);
                const __half l0 = __float2half_rn(o0 - __half2float(h0)), l1 = __float2half_rn(o1 - __half2float(h1));
                hw[p] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
                lw[p] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
            }
            const uint32_t off = sw_off(kRows, r, lane);
            *reinterpret_cast<uint4 *>(sm + oQhi + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4 *>(sm + oQlo + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            __syncwarp();
        }
    }

    fence_smem_to_async_proxy();  // (f16: the TMA engine writes where the staging rows were)
    __syncthreads();  // the staging area becomes the K tile

    // ---- per-thread share of a packed tile: position tid / 8, coordinates 32 (tid % 8) .. + 31 ----
    const int my_row = tid >> 3, my_c = tid & 7;
    const size_t seq_rows = (size_t)pa.seq * a.seq_stride_rows;
    uint32_t pk[4], pv[4];
    float pn = 0.f;
    // f32: the thread's 128 bytes of a K row or of a V row (one buffer: K of this tile until it is split, then
    // V of this tile, then K of the next one)
    [[maybe_unused]] float4 pf[kVRows32 ? 8 : 1];
    [[maybe_unused]] auto fetch_f32 = [&](int tile, bool v_side) {
        const int pos = min(c0 + tile * kTK + my_row, a.n_ctx - 1);
        const size_t row = seq_rows + (size_t)pos * a.n_kv + kv;
        const float4 *src = reinterpret_cast<const float4 *>((v_side ? a.v_rows : a.k_rows) + row * 1024) + 8 * my_c;
#pragma unroll
        for (int i = 0; i < (kVRows32 ? 8 : 1); i++) pf[i] = __ldg(src + i);
    };
    // f32: split the buffer into f16 hi + lo and store both as four 16-byte chunks of a tile row; rows at or past
    // `end` are stored as zeros (they may hold anything, and 0 * Inf would poison the accumulators)
    [[maybe_unused]] auto split_store_f32 = [&](uint8_t *tile_hi, uint8_t *tile_lo, int rows, int row_hi, int row_lo, bool live) {
#pragma unroll
        for (int j = 0; j < (kVRows32 ? 4 : 0); j++) {
            const float x[8] = {pf[2 * j].x, pf[2 * j].y, pf[2 * j].z, pf[2 * j].w, pf[2 * j + 1].x, pf[2 * j + 1].y, pf[2 * j + 1].z, pf[2 * j + 1].w};
            uint32_t h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float x0 = live ? x[2 * e] : 0.f, x1 = live ? x[2 * e + 1] : 0.f;
                const __half2 hv = __floats2half2_rn(x0, x1);
                const float2 hf = __half22float2(hv);
                const __half2 lv = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
                h[e] = *reinterpret_cast<const uint32_t *>(&hv);
                l[e] = *reinterpret_cast<const uint32_t *>(&lv);
            }
            *reinterpret_cast<uint4 *>(tile_hi + sw_off(rows, row_hi, 4 * my_c + j)) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4 *>(tile_lo + sw_off(rows, row_lo, 4 * my_c + j)) = make_uint4(l[0], l[1], l[2], l[3]);
        }
    };
    auto fetch = [&](int tile) {
        if constexpr (kF16) return;
        if constexpr (kF32) {
            fetch_f32(tile, false);
            return;
        }
        const int pos = min(c0 + tile * kTK + my_row, a.n_ctx - 1);
        const size_t row = seq_rows + (size_t)pos * a.n_kv + kv;
        const uint8_t *kr = a.k_rows + row * kRowBytes, *vr = a.v_rows + row * kRowBytes;
        if constexpr (VF32) {  // only the K row is packed (vr is not used: the V row is fetched as floats below)
            if constexpr (BITS == 4) {
                const uint4 x = __ldg(reinterpret_cast<const uint4 *>(kr) + my_c);
                pk[0] = x.x; pk[1] = x.y; pk[2] = x.z; pk[3] = x.w;
            } else {
                const uint32_t *k3 = reinterpret_cast<const uint32_t *>(kr) + 3 * my_c;
                pk[0] = __ldg(k3); pk[1] = __ldg(k3 + 1); pk[2] = __ldg(k3 + 2); pk[3] = 0;
            }
        } else if constexpr (BITS == 4) {
            const uint4 x = __ldg(reinterpret_cast<const uint4 *>(kr) + my_c), y = __ldg(reinterpret_cast<const uint4 *>(vr) + my_c);
            pk[0] = x.x; pk[1] = x.y; pk[2] = x.z; pk[3] = x.w;
            pv[0] = y.x; pv[1] = y.y; pv[2] = y.z; pv[3] = y.w;
        } else if constexpr (BITS == 3) {
            const uint32_t *k3 = reinterpret_cast<const uint32_t *>(kr) + 3 * my_c, *v3 = reinterpret_cast<const uint32_t *>(vr) + 3 * my_c;
            pk[0] = __ldg(k3); pk[1] = __ldg(k3 + 1); pk[2] = __ldg(k3 + 2); pk[3] = 0;
            pv[0] = __ldg(v3); pv[1] = __ldg(v3 + 1); pv[2] = __ldg(v3 + 2); pv[3] = 0;
        } else {  // 2 bit: 32 coordinates are 8 bytes
            const uint2 x = __ldg(reinterpret_cast<const uint2 *>(kr) + my_c), y = __ldg(reinterpret_cast<const uint2 *>(vr) + my_c);
            pk[0] = x.x; pk[1] = x.y; pk[2] = pk[3] = 0;
            pv[0] = y.x; pv[1] = y.y; pv[2] = pv[3] = 0;
        }
        if (tid < (VF32 ? kTK : 2 * kTK)) {
            const int p2 = min(c0 + tile * kTK + (tid & (kTK - 1)), a.n_ctx - 1);
            pn = __ldg((tid < kTK ? a.k_norms : a.v_norms) + seq_rows + (size_t)p2 * a.n_kv + kv);
        }
        if constexpr (VF32) fetch_f32(tile, true);
    };
    auto widen = [&](uint32_t (&w)[4]) {
        if constexpr (BITS == 3) {
            const uint32_t u0 = w[0], u1 = w[1], u2 = w[2];
            w[0] = expand24u(u0);
            w[1] = expand24u(__funnelshift_r(u0, u1, 24));
            w[2] = expand24u(__funnelshift_r(u1, u2, 16));
            w[3] = expand24u(u2 >> 8);
        } else if constexpr (BITS == 2) {  // sixteen indices per word -> two words of eight nibbles
            const uint32_t u0 = w[0], u1 = w[1];
            w[0] = expand16u(u0);
            w[1] = expand16u(u0 >> 16);
            w[2] = expand16u(u1);
            w[3] = expand16u(u1 >> 16);
        }
    };
    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        int polls = 0;
        while (!mbar_try_wait(bar, parity)) {
            if (++polls > kWaitPolls) {  // never expected; leave a mark and go on rather than hang
                if (lane == 0) raise_error(pa.err_flag, 4);
                break;
            }
        }
    };

    // this thread's query row (warps 0-3): causal limit, running reference and sum
    const int my_q = (warp & 3) * 32 + lane;
    const int lim = (warp < 4 && my_q < n_rows) ? pa.pos0 + tok0 + my_q / NREP + 1 : 0;
    float R = -CUDART_INF_F, lsum = 0.f;
    const uint32_t tab = (uint32_t)__half_as_ushort(ss.table[lane & 15]) | ((uint32_t)__half_as_ushort(ss.table_lo[lane & 15]) << 16);
    const uint32_t idesc_s = umma_idesc_f16(kRows, kTK, 0, 0), idesc_s2 = umma_idesc_f16(kRows, kKRows, 0, 0);
    const uint32_t idesc_o = umma_idesc_f16(kRows, kHd, 0, 1);

    // f16: one thread has the TMA engine copy tile `tile` (32 rows x 512 bytes of K and of V, as
    // 16 boxes of 16 rows x 128 bytes) into stage st; completion on bar_t[st].
    auto issue_tma = [&](int tile, int st) {
        const uint32_t bar = bar_t + (uint32_t)st * 8u, dstk = base + oKhi + (uint32_t)st * 2u * kKVTile, dstv = dstk + kKVTile;
        mbar_expect_tx(bar, 2 * kKVTile);
        const int gpos = a.layer_pos0 + pa.seq * a.n_ctx + c0 + tile * kTK;
#pragma unroll
        for (int sl = 0; sl < 4; sl++)
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                tma_tile_x(dstk + sl * kKVSlab + hf * 2048, &tm_k, sl * 128, kv, gpos + 16 * hf, bar);
                tma_tile_x(dstv + sl * kKVSlab + hf * 2048, &tm_v, sl * 128, kv, gpos + 16 * hf, bar);
            }
    };
    // Packed (or f32) caches: K of tile t + 1 is dequantized right after the O products of tile t are issued, so
    // that it runs under them (the K tile is free once S of tile t is complete, which the softmax has waited for);
    // the norms of the tile travel with it.
    [[maybe_unused]] auto dequant_k = [&](int tile) {
        if constexpr (kF32) {
            split_store_f32(sm + oKhi, sm + oKhi, kKRows, my_row, my_row + 32, c0 + tile * kTK + my_row < c1);
            fetch_f32(tile, true);  // this tile's V rows travel while the S products are issued
        } else if constexpr (!kF16) {
            widen(pk);
            dequant_store_shfl<kLoTiles>(pk, tab, sm + oKhi, sm + oKhi, kKRows, my_row, my_row + 32, 4 * my_c);
            if (tid < kTK) ss.kn[tid] = pn;
            else if (tid < 2 * kTK) ss.lv[tid - kTK] = VF32 ? 0.f : fast_log2(fmaxf(pn, 1e-30f));
        }
        fence_smem_to_async_proxy();
    };
    if constexpr (kF16) {
        if (tid == 0 && n_tiles > 0) issue_tma(0, 0);
    } else {
        if (n_tiles > 0) {
            fetch(0);
            dequant_k(0);
        }
        __syncthreads();
    }
    for (int tile = 0; tile < n_tiles; tile++) {
        const uint32_t parity = (uint32_t)tile & 1u;
        const int st = kF16 ? (tile & 1) : 0;
        const uint32_t k_off = kF16 ? oKhi + (uint32_t)st * 2u * kKVTile : oKhi, v_off = kF16 ? k_off + kKVTile : oVhi;
        if constexpr (kF16) {
            // ---- 1. the next tile starts travelling (its stage was released when bar_o was awaited);
            // this tile has landed; rows past the chunk's end may hold anything and are zeroed
            if (tid == 0 && tile + 1 < n_tiles) issue_tma(tile + 1, st ^ 1);
            wait_bar(bar_t + (uint32_t)st * 8u, (uint32_t)(tile >> 1) & 1u);
            const int valid = c1 - (c0 + tile * kTK);
            if (valid < kTK) {
                for (int i = tid; i < 2 * 4 * kTK * 8; i += kUT) {
                    const int tl = i >> 10, slab = (i >> 8) & 3, r = (i >> 3) & 31, c = i & 7;
                    if (r >= valid) *reinterpret_cast<uint4 *>(sm + k_off + tl * kKVTile + slab * kKVSlab + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            fence_smem_to_async_proxy();
            __syncthreads();
        }  // (packed and f32 caches: K of this tile was dequantized at the end of the previous iteration)

        // ---- 2. S = Q . K^T, and V is dequantized while it runs ---------------------------------------
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                const uint32_t qo = (uint32_t)(ks >> 2) * kQSlab + (uint32_t)(ks & 3) * 32u;
                const uint32_t ko = (uint32_t)(ks >> 2) * kKSlab + (uint32_t)(ks & 3) * 32u;
                const uint64_t qh = umma_smem_desc(base + oQhi + qo, 16, 1024, kUmmaSwizzle128);
                const uint64_t ql = umma_smem_desc(base + oQlo + qo, 16, 1024, kUmmaSwizzle128);
                const uint64_t kd = umma_smem_desc(base + k_off + ko, 16, 1024, kUmmaSwizzle128);
                umma_f16_ss(tmem + kColS, qh, kd, idesc_s2, ks > 0);  // columns 0-31: q_hi k_hi, 32-63: q_hi k_lo
                umma_f16_ss(tmem + kColS, ql, kd, idesc_s, true);     // columns 0-31 += q_lo k_hi
            }
            umma_commit(bar_s);
        }
        __syncwarp();
        if constexpr (!kF16) {
            // the previous tile's O products read the V tiles and the P buffers and write O: they must be complete
            // before V is overwritten here and before the softmax below rescales O or rewrites P
            if (tile > 0) {
                wait_bar(bar_o, (uint32_t)(tile - 1) & 1u);
                tc_fence_after_sync();
            }
        }
        if constexpr (kVRows32) {
            split_store_f32(sm + oVhi, sm + oVlo, kTK, my_row, my_row, c0 + tile * kTK + my_row < c1);
            if (tile + 1 < n_tiles) fetch(tile + 1);
            fence_smem_to_async_proxy();
        } else if constexpr (!kF16) {
            widen(pv);
            dequant_store_shfl<kLoTiles>(pv, tab, sm + oVhi, sm + oVlo, kTK, my_row, my_row, 4 * my_c);
            if (tile + 1 < n_tiles) fetch(tile + 1);
            fence_smem_to_async_proxy();
        }

        // ---- 3. softmax: thread = query row ---------------------------------------------------------
        if (warp < 4) {
            wait_bar(bar_s, parity);
            tc_fence_after_sync();
            uint32_t sr[32];
            tmem_ld32(my_tmem + kColS, sr);
            if constexpr (kLoTiles) {
                uint32_t s2[32];
                tmem_ld32(my_tmem + kColS + 32, s2);
#pragma unroll
                for (int j = 0; j < 32; j++) sr[j] = __float_as_uint(__uint_as_float(sr[j]) + __uint_as_float(s2[j]));
            }
            const int pb = c0 + tile * kTK;
            float t[32];
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float s = __uint_as_float(sr[j]) * ss.kn[j];
                sr[j] = __float_as_uint(s);
                const int p = pb + j;
                t[j] = (p < c1 && p < lim) ? s + ss.lv[j] : -CUDART_INF_F;
                mx = fmaxf(mx, t[j]);
            }
            // lazy reference: move it only when this row's maximum ran ahead by more than kLazy
            const bool move = mx > -CUDART_INF_F && (R == -CUDART_INF_F || mx > R + kLazy);
            if (__any_sync(0xffffffffu, move)) {  // tensor-memory traffic is warp-collective
                const float newR = move ? mx : R;
                const float f = (move && R > -CUDART_INF_F) ? fast_exp2(R - newR) : (move ? 0.f : 1.f);
                lsum *= f;
                for (int b = 0; b < 8; b++) {
                    uint32_t o[32];
                    tmem_ld32(my_tmem + kColO + 32 * b, o);
#pragma unroll
                    for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
                    tmem_st32(my_tmem + kColO + 32 * b, o);
                }
                tmem_wait_st();
                R = newR;
            }
            const float ref = R > -CUDART_INF_F ? R : 0.f;
            // weights: chunk c = positions 8c .. 8c+7 -> 16 bytes at c * 2048 + (row / 8) * 128 + (row % 8) * 16
            uint8_t *p_hi = sm + oPhi + (my_q >> 3) * 128 + (my_q & 7) * 16, *p_lo = sm + oPlo + (my_q >> 3) * 128 + (my_q & 7) * 16;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t hw[4], lw[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int j = 8 * c + 2 * e;
                    const float w0 = fast_exp2(t[j] - ref) * kPScale, w1 = fast_exp2(t[j + 1] - ref) * kPScale;
                    if (t[j] > -CUDART_INF_F) lsum += fast_exp2(__uint_as_float(sr[j]) - ref);
                    if (t[j + 1] > -CUDART_INF_F) lsum += fast_exp2(__uint_as_float(sr[j + 1]) - ref);
                    const __half2 h = __floats2half2_rn(w0, w1);
                    const float2 hf = __half22float2(h);
                    const __half2 l = __floats2half2_rn(w0 - hf.x, w1 - hf.y);
                    hw[e] = *reinterpret_cast<const uint32_t *>(&h);
                    lw[e] = *reinterpret_cast<const uint32_t *>(&l);
                }
                *reinterpret_cast<uint4 *>(p_hi + c * kPChunk) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                *reinterpret_cast<uint4 *>(p_lo + c * kPChunk) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            }
            tc_fence_before_sync();
            fence_smem_to_async_proxy();
        }
        __syncthreads();

        // ---- 4. O += P . V ----------------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 2; kk++) {
                const uint64_t ph = umma_smem_desc(base + oPhi + kk * 2 * kPChunk, kPChunk, 128, kUmmaSwizzleNone);
                const uint64_t pl = umma_smem_desc(base + oPlo + kk * 2 * kPChunk, kPChunk, 128, kUmmaSwizzleNone);
                const uint64_t vh = umma_smem_desc(base + v_off + kk * 2048, kKVSlab, 1024, kUmmaSwizzle128);
                umma_f16_ss(tmem + kColO, ph, vh, idesc_o, true);
                umma_f16_ss(tmem + kColO, pl, vh, idesc_o, true);
                if constexpr (kLoTiles) {
                    const uint64_t vl = umma_smem_desc(base + oVlo + kk * 2048, kKVSlab, 1024, kUmmaSwizzle128);
                    umma_f16_ss(tmem + kColO, ph, vl, idesc_o, true);
                }
            }
            umma_commit(bar_o);
        }
        __syncwarp();
        if constexpr (kF16) {
            wait_bar(bar_o, parity);  // everybody: the tiles and the P buffers may be overwritten, O may be rescaled
            tc_fence_after_sync();
        } else {
            if (tile + 1 < n_tiles) dequant_k(tile + 1);  // under the O products just issued
            __syncthreads();
        }
    }
    if constexpr (!kF16) {
        if (n_tiles > 0) {  // the last tile's O products
            wait_bar(bar_o, (uint32_t)(n_tiles - 1) & 1u);
            tc_fence_after_sync();
        }
    }

    // ---- epilogue: thread = query row ------------------------------------------------------------------
    if (warp < 4) {  // every lane takes part in the warp-collective tensor-memory loads, rows past the block only skip the stores
        const bool real = my_q < n_rows;
        const size_t out_row = real ? (size_t)(tok0 + my_q / NREP) * a.n_head + kv * NREP + my_q % NREP : 0;
        const float unscale = 1.0f / (kPScale * (kVPlanar ? pa.lut_alpha : 1.0f));  // (raw V rows carry no table scale)
        const bool whole = pa.n_chunks == 1;
        const float mul = whole ? (lsum > 0.f ? unscale / lsum : 0.f) : unscale;
        float *dst = whole ? a.out + out_row * kHd : pa.scratch + (out_row * pa.n_chunks + chunk) * (kHd + 2);
        // 32 rows x 32 columns at a time through a padded shared-memory block, so that the global
        // stores of a warp cover one row's 128 bytes instead of 32 rows' 8 bytes
        float *stg = reinterpret_cast<float *>(sm + oKhi) + (warp & 3) * (32 * 33);
        const int wrow0 = (warp & 3) * 32;
        for (int b = 0; b < 8; b++) {
            uint32_t o[32];
            tmem_ld32(my_tmem + kColO + 32 * b, o);
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const int d = 32 * b + j;
                float o0 = __uint_as_float(o[j]) * mul, o1 = __uint_as_float(o[j + 1]) * mul;
                if (whole && kVPlanar) {
                    float r0, r1;
                    givens_inv(o0, o1, ss.givens[d], ss.givens[d + 1], r0, r1);
                    o0 = r0;
                    o1 = r1;
                }
                stg[lane * 33 + j] = o0;
                stg[lane * 33 + j + 1] = o1;
            }
            __syncwarp();
            for (int rr = 0; rr < 32; rr++) {
                const int q = wrow0 + rr;
                if (q >= n_rows) break;
                const size_t orow = (size_t)(tok0 + q / NREP) * a.n_head + kv * NREP + q % NREP;
                float *drow = whole ? a.out + orow * kHd : pa.scratch + (orow * pa.n_chunks + chunk) * (kHd + 2);
                drow[32 * b + lane] = stg[rr * 33 + lane];
            }
            __syncwarp();
        }
        if (real && !whole) {
            dst[kHd] = R;
            dst[kHd + 1] = lsum;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// One CTA of 128 threads per output row: merge the chunks' triples, rotate back, write.
__global__ void __launch_bounds__(128) prefill_umma_merge_kernel(const float *scratch, const float *givens, int n_chunks, float *out) {
    const size_t row = blockIdx.x;
    const int pr = threadIdx.x;
    const float *basep = scratch + row * n_chunks * (kHd + 2);
    float M = -CUDART_INF_F;
    for (int c = 0; c < n_chunks; c++) M = fmaxf(M, basep[(size_t)c * (kHd + 2) + kHd]);
    float a0 = 0.f, a1 = 0.f, Ls = 0.f;
    for (int c = 0; c < n_chunks; c++) {
        const float *p = basep + (size_t)c * (kHd + 2);
        const float m = p[kHd];
        if (!(m > -CUDART_INF_F)) continue;
        const float f = exp2f(m - M);
        const float2 v = *reinterpret_cast<const float2 *>(p + 2 * pr);
        a0 = fmaf(v.x, f, a0);
        a1 = fmaf(v.y, f, a1);
        Ls = fmaf(p[kHd + 1], f, Ls);
    }
    const float inv = Ls > 0.f ? 1.0f / Ls : 0.f;
    float o0 = a0 * inv, o1 = a1 * inv;
    if (givens) givens_inv(a0 * inv, a1 * inv, givens[2 * pr], givens[2 * pr + 1], o0, o1);  // planar V only
    *reinterpret_cast<float2 *>(out + row * kHd + 2 * pr) = make_float2(o0, o1);
}

template <int BITS, int NREP, bool VF32 = false>
bk_status launch_umma_one(bk_ctx *ctx, const PrefillUArgs &pa) {
    static std::atomic<bool> configured[64] = {};  // per device; racing first calls set the same attribute
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, BK_ERR_UNSUPPORTED, "prefill: device index above 63");
    if (!configured[dev].load()) {
        BK_CUDA(ctx, cudaFuncSetAttribute(prefill_umma_kernel<BITS, NREP, VF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUmmaSmem));
        configured[dev].store(true);
    }
    const int grid = pa.n_blocks * pa.d.n_kv * pa.n_chunks;
    if (!pa.d.h_tmap_k || !pa.d.h_tmap_v) return fail(ctx, BK_ERR_INVALID, "prefill: the cache has no tensor maps");
    prefill_umma_kernel<BITS, NREP, VF32><<<grid, kUT, kUmmaSmem, ctx->stream>>>(pa, *static_cast<const CUtensorMap *>(pa.d.h_tmap_k),
                                                                          *static_cast<const CUtensorMap *>(pa.d.h_tmap_v));
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    if (pa.n_chunks > 1) {
        prefill_umma_merge_kernel<<<pa.n_tokens * pa.d.n_head, 128, 0, ctx->stream>>>(pa.scratch, (BITS == 16 || BITS == 32 || VF32) ? nullptr : pa.d.givens,
                                                                                      pa.n_chunks, pa.d.out);
        ctx->launches++;
        BK_CUDA(ctx, cudaGetLastError());
    }
    return BK_OK;
}

}  // namespace

bool prefill_umma_supported(const DecodeArgs &a) {
    const int n_rep = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    const bool planar = a.k_kind == ROW_PLANAR && a.v_kind == ROW_PLANAR && (a.bits == 4 || a.bits == 3 || a.bits == 2);
    const bool f16 = a.k_kind == ROW_F16 && a.v_kind == ROW_F16 && a.k_row_bytes == 512 && a.v_row_bytes == 512;
    const bool f32 = a.k_kind == ROW_F32 && a.v_kind == ROW_F32 && a.k_row_bytes == 1024 && a.v_row_bytes == 1024;
    const bool k_only = a.k_kind == ROW_PLANAR && a.v_kind == ROW_F32 && (a.bits == 4 || a.bits == 3) && a.v_row_bytes == 1024;
    return (planar || f16 || f32 || k_only) && a.h_tmap_k && a.h_tmap_v && (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 6);
}

bk_status launch_prefill_umma(bk_ctx *ctx, const DecodeArgs &a, int seq, int pos0, int n_tokens, float alpha) {
    if (n_tokens <= 0) return BK_OK;
    const int n_rep = a.n_head / a.n_kv;
    PrefillUArgs pa{};
    pa.d = a;
    pa.seq = seq;
    pa.pos0 = pos0;
    pa.n_tokens = n_tokens;
    pa.tq = kRows / n_rep;
    pa.n_blocks = (n_tokens + pa.tq - 1) / pa.tq;
    pa.lut_alpha = alpha;
    pa.err_flag = ctx->d_err;
    const int vis = pos0 + n_tokens;
    int chunks = (4 * ctx->n_sms + pa.n_blocks * a.n_kv - 1) / (pa.n_blocks * a.n_kv);  // about four CTAs per SM: the causal triangle leaves them unequal
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
#define BK_PU_CASE(R)                                                                            \
    case R:                                                                                      \
        if (a.k_kind == ROW_F16) return launch_umma_one<16, R>(ctx, pa);                         \
        if (a.k_kind == ROW_F32) return launch_umma_one<32, R>(ctx, pa);                         \
        if (a.v_kind == ROW_F32) return a.bits == 3 ? launch_umma_one<3, R, true>(ctx, pa) : launch_umma_one<4, R, true>(ctx, pa); \
        if (a.bits == 2) return launch_umma_one<2, R>(ctx, pa);                                  \
        return a.bits == 3 ? launch_umma_one<3, R>(ctx, pa) : launch_umma_one<4, R>(ctx, pa);
    switch (n_rep) {
        BK_PU_CASE(1)
        BK_PU_CASE(2)
        BK_PU_CASE(4)
        BK_PU_CASE(6)
        default: return fail(ctx, BK_ERR_UNSUPPORTED, "prefill: n_head/n_kv must be 1, 2, 4 or 6");
    }
#undef BK_PU_CASE
}

}  // namespace bk
