// Decode attention over an f16 or an f32 cache (K and V rows of 256 halfs or floats), or 4/3-bit K rows beside
// f32 V rows: tensor-core path.
//
// f16: the stored halfs are MMA operands as they are, so the kernel is the 4-bit one without its
// lookup table: per warp a ring of shared-memory stages, each one tile of 16 positions of one kv
// head (K 8 KiB + V 8 KiB), filled by the TMA engine as eight tiled copies of 16 rows x 128 bytes
// (a 3-D tensor map over [position][kv head][512 B]; four column slabs per row because the
// 128-byte swizzle spans 128 bytes), completion on an mbarrier with a bounded wait.  Fragments
// come out of the swizzled slabs with ldmatrix (conflict-free: the eight rows of a matrix sit in
// eight different 16-byte columns):
//     scores^T[16 pos x 8 heads] = K[16 pos x 256] . Q^T      (A = K via ldmatrix, B = q)
//     out^T[256 x 8 heads]      += V^T[256 x 16 pos] . W      (A = V via ldmatrix.trans, B = weights)
// with mma.sync.m16n8k16, f16 in, f32 accumulate.  K and V are exact as stored; q and the V
// weights (p * 2^14) are each split into f16 hi + lo parts when QSPLIT is set, so both products
// carry about 22 bits; the softmax runs in f32 in the exp2 domain.  Six of the eight MMA columns
// are real heads (the GQA group).
//
// f32 (EB = 4): the same contraction with every stored float split on the fly into f16 hi + lo
// (x = hi + lo to about 22 bits; |x| up to 65504, which activations never approach), three MMAs
// per fragment (hi.hi, lo.hi, hi.lo).  A row is 1 KiB = eight slabs, a tile of 16 positions 16 KiB
// for K and as much for V, so a CTA has six warps with one K and one V buffer each (192 KiB), each
// buffer with its own mbarrier and refilled as soon as its half of the tile is done; a row costs
// a quarter of the instructions per byte of the 4-bit kernel, so six warps keep up with HBM.
// Fragments are read with plain 8-byte (K: two adjacent coordinates of a row) and 4-byte (V: one
// coordinate of two adjacent rows) loads, conflict-free under the 128-byte swizzle.
// K-only planar (KB = -4, -3): the reference's mixed mode, quantized K beside f32 V (src/kvquant.rs:515-543
// with the trailing 'k'; src/gdev.rs:706-717, 770-779).  The K product is the 4-bit kernel's for one row
// block: a 256-entry table of half2(c[lo nibble], c[hi nibble]) per lane (here behind the bookkeeping
// block, its index added to the lane's base), one lookup per packed byte, q Givens-rotated into the rows'
// basis, the row norms (which travel with the K tile) on the scores; the V product is the f32 one.
// Unlike the 4-bit kernel this one also carries what the rounding of the centroids to f16 left over (a second
// half2 in the upper half of each table slot, one more load and one more MMA per fragment): V rows here are
// raw activations, several times larger than dequantized ones, and the 11-bit table alone showed as 2e-3 in
// the output at short contexts; with the remainders the result is within ~1e-5 of the f32 CPU path.
// The CPU path this replaces is src/forward.rs:297-343 (planar and f16 rows, f32 dot, f64 softmax sum)
// and src/forward.rs:344-375 (f32 rows).
//
// Work split, partials and the last-arriver combine are shared with the other decode kernels.
#include <cuda.h>
#include <cuda_fp16.h>

#include <atomic>

#include "bk_decode_common.cuh"
#include "bk_mma_common.cuh"

namespace bk {

namespace {

constexpr int kMaxFW = 12;               // warps per CTA: 12 (f16), 8 of which 6 scan (f32)
constexpr int kTile = 16;                // positions per warp tile (the MMA's M)
constexpr int kSlabBytes = kTile * 128;  // 16 rows x 128 B, 128B-swizzled
constexpr int kMaxStages = 2;
// KB / VB: bytes per stored K / V element (2 = f16, 4 = f32); KB = -4 or -3: K rows in the 4- or 3-bit planar
// format (128 or 96 bytes of indices + a norm, src/kvquant.rs:397-412) beside f32 V rows, the reference's
// K-only mode.
template <int KB, int VB> struct Rows {
    static constexpr bool kPlanarK = KB < 0;
    static constexpr int kBits = kPlanarK ? -KB : 0;
    // f16 + f16: up to two stages per warp, one barrier per stage.  Otherwise: one stage per warp, its K and V
    // halves with a barrier each (bar[warp][0], bar[warp][1]).
    static constexpr bool kSplitHalves = !(KB == 2 && VB == 2);
    static constexpr int kFW = kSplitHalves ? 8 : 12;        // warps in the CTA
    static constexpr int kScanW = kSplitHalves ? 6 : 12;     // of which this many scan (six buffers of 32 KiB fit)
    static constexpr int kFT = kFW * 32;
    static constexpr int kSlabsK = kPlanarK ? 1 : KB * 2;    // 128-byte column slabs per row: 4 (f16), 8 (f32), 1 (planar)
    static constexpr int kSlabsV = VB * 2;
    static constexpr int kHalfK = kPlanarK ? 3072 : kSlabsK * kSlabBytes;  // planar: the tile, then its norms (1 KiB slot)
    static constexpr int kHalfV = kSlabsV * kSlabBytes;
    static constexpr int kStageBytes = kHalfK + kHalfV;
};
constexpr uint32_t kLutBytes = 65536;    // planar K: 256 entries x 256 B, one word per lane (as in the 4-bit kernel)
constexpr int kHeadStride = 276;         // floats per head in the warp-merge area (bank-conflict free)
constexpr float kWScale = 16384.0f;      // 2^14: V weights are stored as f16 in (0, 2^14]

struct Other {
    uint2 q_hi_frag[16][32], q_lo_frag[16][32];  // q as B fragments: [k-step][lane]
    float sq[8 * kHd];                   // q of the group while it is roped
    float new_row[2][kHd];               // the newest token's k and v of this kv head (fused append)
    float2 rope_row[kHd / 2];            // (cos, sin) of the q position
    float qw[kHd];                       // q RMSNorm weight (layer form of the step)
    float givens[kHd];                   // planar K: (cos, sin) pairs
    float book[16];                      // planar K: unscaled centroids (fused append)
    float m_w[kMaxFW][8], l_w[kMaxFW][8];
    float M[8], L[8];
    int last;
    unsigned long long bar[kMaxFW][kMaxStages];
    unsigned long long fin_bar[2];       // the split-K combine's two streaming rounds
};

// f32 -> f16 hi + lo for two values at once: hi = rn(x), lo = rn(x - hi).
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// Eight 3-bit indices in the low 24 bits of y -> eight nibbles.
__device__ __forceinline__ uint32_t expand24(uint32_t y) {
    y &= 0x00ffffffu;
    y += (y & 0x00fff000u) * 15u;   // upper four indices up by 4 bits
    y += (y & 0x0fc00fc0u) * 3u;    // upper two of every four up by 2
    y += (y & 0x38383838u);         // upper one of every two up by 1
    return y;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Table lookup of packed byte K (0..3) of word x in a table that starts anywhere: the byte moves to bits 8..15
// and is added to the lane's base address (table + 4 * lane); the entry's rounding remainder (the slot's upper
// half) comes with it.
template <int K>
__device__ __forceinline__ void lutx2(uint32_t x, uint32_t lane_base, uint32_t &v, uint32_t &rem) {
    uint32_t off;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(off) : "r"(x), "r"(0u), "n"(0x4404 | (K << 4)));
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(off + lane_base));
    asm volatile("ld.shared.b32 %0, [%1+128];\n" : "=r"(rem) : "r"(off + lane_base));
}

template <int KB, int VB, int NREP, bool QSPLIT>
__global__ void __launch_bounds__(Rows<KB, VB>::kFT, 1)
decode_f16_mma_kernel(DecodeArgs a, DecodeMeta meta, float lut_alpha, uint32_t smem_bytes, int *err_flag,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    using R = Rows<KB, VB>;
    constexpr int kFW = R::kFW, kFT = R::kFT, kSlabsK = R::kSlabsK, kSlabsV = R::kSlabsV, kScanW = R::kScanW;
    constexpr int kHalfK = R::kHalfK, kHalfV = R::kHalfV, kStageBytes = R::kStageBytes;
    constexpr bool kSplit = R::kSplitHalves, kPlanarK = R::kPlanarK;
    constexpr int kBits = R::kBits, kRowK = kPlanarK ? 32 * kBits : 256 * KB, kRowV = 256 * VB;
    [[maybe_unused]] constexpr int kKTile = kTile * kRowK;  // planar K: bytes of a tile (2048 or 1536)
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    // ---- shared-memory layout: bookkeeping first, then the ring on a 1 KiB boundary ----------
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    Other &o = *reinterpret_cast<Other *>(smem_raw);
    // planar K: the lookup table follows the bookkeeping block (256-byte aligned), the ring follows the table
    const uint32_t lut_addr = (base + (uint32_t)sizeof(Other) + 255u) & ~255u;
    const uint32_t ring0 = ((kPlanarK ? lut_addr + kLutBytes : base + (uint32_t)sizeof(Other)) + 1023u) & ~1023u;
    [[maybe_unused]] const uint32_t lane_base = lut_addr + (uint32_t)(lane << 2);
    const uint32_t ring_end = base + smem_bytes;
    const int n_stages = ring_end > ring0 ? min((int)((ring_end - ring0) / (uint32_t)(kScanW * kStageBytes)), kSplit ? 1 : kMaxStages) : 0;
    if (n_stages < 1) {  // never expected (the host checks the size): report, do not run
        if (tid == 0) raise_error(err_flag, 2);
        asm volatile("griddepcontrol.wait;\n" ::: "memory");  // keep the stream's kernel order intact
        return;
    }
    const uint32_t bar0 = base + (uint32_t)offsetof(Other, bar) + (uint32_t)(warp * kMaxStages) * 8u;
    if (lane < kMaxStages) mbar_init(bar0 + lane * 8u, 1);
    if (tid < 2) mbar_init(base + (uint32_t)offsetof(Other, fin_bar) + tid * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    __syncthreads();

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
    const int gpos0 = a.layer_pos0 + meta.seq_id[s] * a.n_ctx + p0;  // position index in the tensor map

    auto stage_of = [&](int st) -> uint32_t { return ring0 + (uint32_t)(warp * n_stages + st) * kStageBytes; };
    auto issue_tile = [&](int tile, int st) {  // f16 + f16: a whole stage on one barrier
        if (lane == 0) {
            const uint32_t bar = bar0 + (uint32_t)st * 8u, dst = stage_of(st);
            mbar_expect_tx(bar, kStageBytes);
            const int pos = gpos0 + tile * kTile;
#pragma unroll
            for (int sl = 0; sl < kSlabsK; sl++) tma_tile_x(dst + sl * kSlabBytes, &tm_k, sl * 128, kv, pos, bar);
#pragma unroll
            for (int sl = 0; sl < kSlabsV; sl++) tma_tile_x(dst + kHalfK + sl * kSlabBytes, &tm_v, sl * 128, kv, pos, bar);
        }
    };
    // split form: one half (0 = K, 1 = V) of the warp's single stage, on that half's own barrier
    const uint32_t nb_k = (uint32_t)(kTile * 4 * a.n_kv);  // planar K: the norms of 16 positions, every kv head
    auto issue_half = [&](int tile, int half) {
        if (lane == 0) {
            const uint32_t bar = bar0 + (uint32_t)half * 8u, dst = stage_of(0) + (uint32_t)(half * kHalfK);
            const int pos = gpos0 + tile * kTile;
            if (half == 0) {
                if constexpr (kPlanarK) {
                    mbar_expect_tx(bar, kKTile + nb_k);
                    tma_tile_x(dst, &tm_k, 0, kv, pos, bar);
                    tma_bulk(dst + kSlabBytes, a.k_norms + seq_rows + (size_t)(p0 + tile * kTile) * a.n_kv, nb_k, bar);
                } else {
                    mbar_expect_tx(bar, kHalfK);
#pragma unroll
                    for (int sl = 0; sl < kSlabsK; sl++) tma_tile_x(dst + sl * kSlabBytes, &tm_k, sl * 128, kv, pos, bar);
                }
            } else {
                mbar_expect_tx(bar, kHalfV);
#pragma unroll
                for (int sl = 0; sl < kSlabsV; sl++) tma_tile_x(dst + sl * kSlabBytes, &tm_v, sl * 128, kv, pos, bar);
            }
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

    // ---- constant tables first: with programmatic dependent launch this overlaps the previous
    // kernel's tail.  q, the newest row and the split-K scratch are read after the wait.
    if (!a.no_rope) {
        const int half = a.n_rot >> 1;
        const float2 *cs = a.rope + (size_t)meta.q_pos[s] * half;
        for (int i = tid; i < half; i += kFT) o.rope_row[i] = cs[i];
    }
    if (a.q_norm_w)
        for (int i = tid; i < kHd; i += kFT) o.qw[i] = a.q_norm_w[i];
    if constexpr (kPlanarK) {
        for (int i = tid; i < kHd; i += kFT) o.givens[i] = a.givens[i];
        constexpr int kIdxMask = (1 << (kPlanarK ? kBits : 1)) - 1;
        if (tid < 16) o.book[tid] = tid <= kIdxMask ? a.book[tid] : 0.f;
        // the lookup table: entry e -> half2(alpha * c[low nibble], alpha * c[high nibble]), one copy per lane
        uint8_t *lut_ptr = smem_raw + (lut_addr - base);
        const float c_lo = a.book[lane & kIdxMask] * lut_alpha;
        for (int e = warp; e < 256; e += kFW) {
            const float lo = __shfl_sync(0xffffffffu, c_lo, e & kIdxMask), hi = __shfl_sync(0xffffffffu, c_lo, (e >> 4) & kIdxMask);
            const __half2 hv = __floats2half2_rn(lo, hi);
            const float2 hf = __half22float2(hv);
            *reinterpret_cast<__half2 *>(lut_ptr + e * 256 + lane * 4) = hv;
            // the upper half of the slot: what the rounding to f16 left over (the V rows of this mode are raw
            // activations, so the scores need more than the table's 11 bits; see compute_scores)
            *reinterpret_cast<__half2 *>(lut_ptr + e * 256 + 128 + lane * 4) = __floats2half2_rn(lo - hf.x, hi - hf.y);
        }
    }
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // the counter set of the next launch: whatever the launch before the previous one left there goes now
    if (blockIdx.x == 0 && a.counters_other)
        for (int i = tid; i < a.other_n; i += blockDim.x) a.counters_other[i] = 0;
    // q first: its loads are in flight before the tile copies below fill the memory system's queues
    constexpr int kQPer = (NREP * kHd + kFT - 1) / kFT;
    float q_reg[kQPer];
    {
        const float *q = a.q + ((size_t)meta.slot[s] * a.n_head + (size_t)kv * NREP) * a.q_stride;
#pragma unroll
        for (int u = 0; u < kQPer; u++) {
            const int i = tid + u * kFT;
            q_reg[u] = i < NREP * kHd ? __ldg(q + (size_t)(i >> 8) * a.q_stride + (i & 255)) : 0.f;
        }
    }

    // ---- fused append: the CTA that scans the last chunk of this kv head stores the head's new K
    // and V rows first, exactly as the append kernel would (src/forward.rs:259-277: rope on K,
    // then f32 -> f16 by the reference's own rounding rule).
    if (a.new_k != nullptr && chunk == n_chunks - 1) {
        __syncthreads();  // the rope row is in shared memory
        if (warp < 2) {
            const float *src = (warp == 0 ? a.new_k : a.new_v) + ((size_t)meta.slot[s] * a.n_kv + kv) * kHd;
            float *sx = o.new_row[warp];
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
            const size_t row = seq_rows + (size_t)(n_pos - 1) * a.n_kv + kv;
            uint8_t *dst = warp == 0 ? a.k_rows_w + row * kRowK : a.v_rows_w + row * kRowV;
            const int eb = warp == 0 ? KB : VB;
            if (eb == 2) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; i++)
                    w[i] = (uint32_t)f32_to_half_ref(sx[lane * 8 + 2 * i]) | ((uint32_t)f32_to_half_ref(sx[lane * 8 + 2 * i + 1]) << 16);
                reinterpret_cast<uint4 *>(dst)[lane] = make_uint4(w[0], w[1], w[2], w[3]);
            } else if (eb == 4) {  // f32 rows are stored as they are (src/forward.rs:279-285)
                reinterpret_cast<float4 *>(dst)[lane] = reinterpret_cast<const float4 *>(sx)[lane];
                reinterpret_cast<float4 *>(dst)[lane + 32] = reinterpret_cast<const float4 *>(sx)[lane + 32];
            } else {  // planar K row: norm, unit vector, Givens rotation, nearest centroid, pack (src/kvquant.rs:397-412)
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
                    constexpr int kB = kPlanarK ? kBits : 4;
                    packed |= (uint64_t)nearest_centroid_fast<kB>(r0, o.book) << (kB * (2 * pr));
                    packed |= (uint64_t)nearest_centroid_fast<kB>(r1, o.book) << (kB * (2 * pr + 1));
                }
                store_group8<(kPlanarK ? kBits : 4)>(dst, lane, packed);
                if (lane == 0) a.k_norms_w[row] = n;
            }
            __threadfence();
            asm volatile("fence.proxy.async;\n" ::: "memory");  // generic-proxy stores before the TMA reads below
        }
        __syncthreads();
    }
    // fill the ring now so that the copies fly during the rest of the set-up
    if constexpr (kSplit) {
        if (warp < kScanW && warp < n_tiles) {
            issue_half(warp, 0);
            issue_half(warp, 1);
        }
    } else {
        for (int st = 0; st < n_stages; st++)
            if (warp + st * kFW < n_tiles) issue_tile(warp + st * kFW, st);
    }

    // ---- q: rope, scale, split into f16 hi/lo, laid out as B fragments ---------------------
    {
        float *sq = o.sq;  // [NREP][256]
#pragma unroll
        for (int u = 0; u < kQPer; u++) {
            const int i = tid + u * kFT;
            if (i < NREP * kHd) sq[i] = q_reg[u];
        }
        __syncthreads();
        if (a.q_norm_w) {  // per-head RMSNorm of q (src/forward.rs:242-243); q is not stored, so a tree sum will do
            if (warp < NREP) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < kHd / 32; j++) {
                    const float x = sq[warp * kHd + lane + 32 * j];
                    ss = fmaf(x, x, ss);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                if (lane == 0) o.M[warp] = 1.0f / sqrtf(ss / (float)kHd + a.eps);
            }
            __syncthreads();
            for (int i = tid; i < NREP * kHd; i += kFT) sq[i] = sq[i] * o.M[i >> 8] * o.qw[i & 255];
            __syncthreads();
        }  // also: the rope row is complete
        if (!a.no_rope) {
            const int half = a.n_rot >> 1;
            for (int i = tid; i < NREP * half; i += kFT) {
                const int r = i / half, j = i - r * half;
                float x0 = sq[r * kHd + j], x1 = sq[r * kHd + j + half];
                rope_pair(x0, x1, o.rope_row[j]);
                sq[r * kHd + j] = x0;
                sq[r * kHd + j + half] = x1;
            }
            __syncthreads();
        }
        // 1/sqrt(hd) * log2(e): the scores come out in the exp2 domain.
        // k-step ks covers coordinates 16 ks .. 16 ks + 15; lane (g, t) holds head g's values at
        // 16 ks + 2t, +1 (b0) and 16 ks + 2t + 8, +9 (b1).
        // Planar K: q is Givens-rotated into the stored rows' basis (src/forward.rs:304), the table's alpha is
        // undone in the scale, and k-step ks = c*8 + w*2 + bp covers coordinates (2t+c)*32 + w*8 + bp*4 + 0..3
        // (the order in which the packed bytes of a row come out of the table).
        const float qscale = rsqrtf((float)kHd) * 1.4426950408889634f / (kPlanarK ? lut_alpha : 1.0f);
        for (int i = tid; i < 16 * 32; i += kFT) {
            const int ks = i >> 5, ln = i & 31, gg = ln >> 2, tt = ln & 3;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (kPlanarK) {
                const int c = ks >> 3, w = (ks >> 1) & 3, bp = ks & 1;
                const int d0 = (2 * tt + c) * 32 + w * 8 + bp * 4;
                if (gg < NREP) {
                    givens_fwd(sq[gg * kHd + d0], sq[gg * kHd + d0 + 1], o.givens[d0], o.givens[d0 + 1], x[0], x[1]);
                    givens_fwd(sq[gg * kHd + d0 + 2], sq[gg * kHd + d0 + 3], o.givens[d0 + 2], o.givens[d0 + 3], x[2], x[3]);
#pragma unroll
                    for (int e = 0; e < 4; e++) x[e] *= qscale;
                }
            } else {
                const int d0 = 16 * ks + 2 * tt;
                if (gg < NREP) {
                    x[0] = sq[gg * kHd + d0] * qscale;
                    x[1] = sq[gg * kHd + d0 + 1] * qscale;
                    x[2] = sq[gg * kHd + d0 + 8] * qscale;
                    x[3] = sq[gg * kHd + d0 + 9] * qscale;
                }
            }
            __half h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                h[e] = __float2half_rn(x[e]);
                l[e] = __float2half_rn(x[e] - __half2float(h[e]));
            }
            auto pack = [](__half lo, __half hi) { return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16); };
            o.q_hi_frag[ks][ln] = make_uint2(pack(h[0], h[1]), pack(h[2], h[3]));
            o.q_lo_frag[ks][ln] = make_uint2(pack(l[0], l[1]), pack(l[2], l[3]));
        }
        __syncthreads();
    }
    const uint32_t qh_addr = base + (uint32_t)offsetof(Other, q_hi_frag) + (uint32_t)lane * 8u;
    const uint32_t ql_addr = base + (uint32_t)offsetof(Other, q_lo_frag) + (uint32_t)lane * 8u;
    auto q_frag = [&](uint32_t addr0, int ks, uint32_t &x, uint32_t &y) {
        asm("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(x), "=r"(y) : "r"(addr0 + (uint32_t)ks * 256u));
    };

    float acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    float M0 = -CUDART_INF_F, M1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    // ldmatrix row addresses of this lane inside a slab.  K (plain): matrices (rows 0-7, chunk c),
    // (rows 8-15, c), (rows 0-7, c+1), (rows 8-15, c+1).  V (transposed): (rows 0-7, c),
    // (rows 0-7, c+1), (rows 8-15, c), (rows 8-15, c+1).  Chunk = 16 bytes = 8 coordinates; the
    // swizzle XORs it with row & 7 = lane & 7.
    const uint32_t key = (uint32_t)(lane & 7);
    const uint32_t k_row_off = (uint32_t)((lane & 7) + ((lane >> 3) & 1) * 8) * 128u, k_csel = (uint32_t)(lane >> 4);
    const uint32_t v_row_off = (uint32_t)((lane & 7) + (lane >> 4) * 8) * 128u, v_csel = (uint32_t)((lane >> 3) & 1);

    // Ragged last tile of the sequence: the rows past its end hold whatever the cache has there, possibly
    // non-finite values, and 0 * Inf would poison the accumulators.  Zero them (one K or V tile at addr).
    auto zero_tail = [&](uint32_t addr, int valid, int n_slabs) {
        for (int i = lane; i < n_slabs * kTile * 8; i += 32) {
            const int slab = i >> 7, r = (i >> 3) & 15, c = i & 7;
            if (r >= valid)
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(addr + (uint32_t)(slab * kSlabBytes + r * 128 + c * 16)), "r"(0u) : "memory");
        }
        __syncwarp();
    };
    // ---- scores^T = K . Q^T for the tile at k_addr, then the online softmax: leaves the V weights (B fragments)
    uint32_t b0 = 0, b1 = 0, b0l = 0, b1l = 0;
    auto compute_scores = [&](int tile, uint32_t k_addr) {
        const int pb = p0 + tile * kTile;
        if constexpr (!kPlanarK)  // (planar rows past the end are finite whatever their bytes; their scores are masked below)
            if (pb + kTile > p1) zero_tail(k_addr, p1 - pb, kSlabsK);
        float sc[4];
        if constexpr (kPlanarK) {
            // the 4-bit kernel's K product for one row block: rows g and g + 8, chunks 2t and 2t + 1 (swizzled),
            // every packed byte one table lookup = two adjacent coordinates; four chains
            float S[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) S[i][0] = S[i][1] = S[i][2] = S[i][3] = 0.f;
            const uint32_t k_row = k_addr + (uint32_t)(g * kRowK);
            // 3 bit: coordinates 64 t .. 64 t + 63 of a row are 24 bytes (the tile is dense and unswizzled), read once
            // as three 8-byte words and widened to words of eight nibbles: [row g / g + 8][c][w]
            [[maybe_unused]] uint32_t k3[2][2][4];
            if constexpr (kBits == 3) {
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint32_t addr = k_row + (uint32_t)(8 * hh * kRowK) + 24 * t;
                    const uint2 u01 = lds64(addr), u23 = lds64(addr + 8), u45 = lds64(addr + 16);
                    k3[hh][0][0] = expand24(u01.x);
                    k3[hh][0][1] = expand24(__funnelshift_r(u01.x, u01.y, 24));
                    k3[hh][0][2] = expand24(__funnelshift_r(u01.y, u23.x, 16));
                    k3[hh][0][3] = expand24(u23.x >> 8);
                    k3[hh][1][0] = expand24(u23.y);
                    k3[hh][1][1] = expand24(__funnelshift_r(u23.y, u45.x, 24));
                    k3[hh][1][2] = expand24(__funnelshift_r(u45.x, u45.y, 16));
                    k3[hh][1][3] = expand24(u45.y >> 8);
                }
            }
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t kg[4], kh[4];
                if constexpr (kBits == 3) {
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        kg[w] = k3[0][c][w];
                        kh[w] = k3[1][c][w];
                    }
                } else {
                    const uint32_t koff = (uint32_t)(((2 * t + c) ^ g) << 4);
                    const uint4 rk_g = lds128(k_row + koff), rk_h = lds128(k_row + 8 * 128 + koff);
                    kg[0] = rk_g.x; kg[1] = rk_g.y; kg[2] = rk_g.z; kg[3] = rk_g.w;
                    kh[0] = rk_h.x; kh[1] = rk_h.y; kh[2] = rk_h.z; kh[3] = rk_h.w;
                }
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const int ks = c * 8 + w * 2;
                    uint32_t qx, qy, a0, a1, a2, a3, r0, r1, r2, r3;
                    // centroid = table value + remainder, q = hi + lo: value.hi, remainder.hi, value.lo
                    lutx2<0>(kg[w], lane_base, a0, r0);
                    lutx2<0>(kh[w], lane_base, a1, r1);
                    lutx2<1>(kg[w], lane_base, a2, r2);
                    lutx2<1>(kh[w], lane_base, a3, r3);
                    q_frag(qh_addr, ks, qx, qy);
                    mma16816(S[c], a0, a1, a2, a3, qx, qy);
                    mma16816(S[2 + c], r0, r1, r2, r3, qx, qy);
                    if (QSPLIT) {
                        q_frag(ql_addr, ks, qx, qy);
                        mma16816(S[2 + c], a0, a1, a2, a3, qx, qy);
                    }
                    lutx2<2>(kg[w], lane_base, a0, r0);
                    lutx2<2>(kh[w], lane_base, a1, r1);
                    lutx2<3>(kg[w], lane_base, a2, r2);
                    lutx2<3>(kh[w], lane_base, a3, r3);
                    q_frag(qh_addr, ks + 1, qx, qy);
                    mma16816(S[2 + c], a0, a1, a2, a3, qx, qy);
                    mma16816(S[c], r0, r1, r2, r3, qx, qy);
                    if (QSPLIT) {
                        q_frag(ql_addr, ks + 1, qx, qy);
                        mma16816(S[c], a0, a1, a2, a3, qx, qy);
                    }
                }
            }
            // the stored rows are unit vectors: their norms scale the scores (src/forward.rs:306)
            float kn0, kn1;
            const uint32_t na = k_addr + (uint32_t)kSlabBytes + (uint32_t)((g * a.n_kv + kv) * 4);  // the norms sit behind the tile's 2 KiB slot
            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(kn0) : "r"(na));
            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(kn1) : "r"(na + (uint32_t)(8 * a.n_kv * 4)));
#pragma unroll
            for (int i = 0; i < 4; i++) sc[i] = ((S[0][i] + S[1][i]) + (S[2][i] + S[3][i])) * ((i >> 1) ? kn1 : kn0);
        } else if constexpr (KB == 2) {
            // four independent accumulator chains
            float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
            float sc2[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                const uint32_t addr = k_addr + (uint32_t)((ks >> 2) * kSlabBytes) + k_row_off + ((((uint32_t)(2 * (ks & 3)) + k_csel) ^ key) << 4);
                uint32_t a0, a1, a2, a3, qx, qy;
                ldmatrix_x4(addr, a0, a1, a2, a3);
                q_frag(qh_addr, ks, qx, qy);
                mma16816((ks & 1) ? sb : sa, a0, a1, a2, a3, qx, qy);
                if (QSPLIT) {
                    q_frag(ql_addr, ks, qx, qy);
                    mma16816((ks & 1) ? sd : sc2, a0, a1, a2, a3, qx, qy);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) sc[i] = (sa[i] + sb[i]) + (sc2[i] + sd[i]);
        } else {
            // k-step ks: coordinates 16 ks .. + 15 = 64 bytes of slab ks / 2.  Lane (g, t) reads the pairs
            // (2t, 2t + 1) and (2t + 8, 2t + 9) of rows g and g + 8: 8-byte loads at chunk (4 (ks & 1) + t / 2
            // (+ 2)) ^ g, half t & 1.  Three chains: hi.hi, lo.hi, hi.lo.
            float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t row_g = k_addr + (uint32_t)(g * 128) + (uint32_t)((t & 1) * 8);
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                const uint32_t slab = row_g + (uint32_t)((ks >> 1) * kSlabBytes);
                const uint32_t c0 = (((uint32_t)(4 * (ks & 1) + (t >> 1))) ^ (uint32_t)g) << 4, c1 = (((uint32_t)(4 * (ks & 1) + 2 + (t >> 1))) ^ (uint32_t)g) << 4;
                float2 x0, x1, x2, x3;
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(x0.x), "=f"(x0.y) : "r"(slab + c0));
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(x1.x), "=f"(x1.y) : "r"(slab + 8 * 128 + c0));
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(x2.x), "=f"(x2.y) : "r"(slab + c1));
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(x3.x), "=f"(x3.y) : "r"(slab + 8 * 128 + c1));
                uint32_t h0, h1, h2, h3, l0_, l1_, l2_, l3_, qx, qy;
                split_pair(x0.x, x0.y, h0, l0_);
                split_pair(x1.x, x1.y, h1, l1_);
                split_pair(x2.x, x2.y, h2, l2_);
                split_pair(x3.x, x3.y, h3, l3_);
                q_frag(qh_addr, ks, qx, qy);
                mma16816(sa, h0, h1, h2, h3, qx, qy);
                mma16816(sb, l0_, l1_, l2_, l3_, qx, qy);
                if (QSPLIT) {
                    q_frag(ql_addr, ks, qx, qy);
                    mma16816(sc2, h0, h1, h2, h3, qx, qy);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) sc[i] = (sa[i] + sc2[i]) + sb[i];
        }
        // ---- online softmax in the exp2 domain ------------------------------------------------
        const bool ok0 = pb + g < p1, ok1 = pb + g + 8 < p1;
        const float t00 = ok0 ? sc[0] : -CUDART_INF_F, t01 = ok0 ? sc[1] : -CUDART_INF_F;
        const float t10 = ok1 ? sc[2] : -CUDART_INF_F, t11 = ok1 ? sc[3] : -CUDART_INF_F;
        float mx0 = fmaxf(t00, t10), mx1 = fmaxf(t01, t11);
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
        const float e00 = fast_exp2(t00 - M0), e01 = fast_exp2(t01 - M1);
        const float e10 = fast_exp2(t10 - M0), e11 = fast_exp2(t11 - M1);
        l0 += e00 + e10;
        l1 += e01 + e11;
        const float w00 = e00 * kWScale, w01 = e01 * kWScale, w10 = e10 * kWScale, w11 = e11 * kWScale;
        const __half2 pl = __floats2half2_rn(w00, w01), ph = __floats2half2_rn(w10, w11);
        b0 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&pl));  // head g; pos 2t, 2t+1
        b1 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph));  // head g; pos 2t+8, 2t+9
        // The weights get a low part as well: V rows are raw activations, and with a peaked softmax
        // over rows of very different size a single f16 weight (11 bits) would show in the output.
        if (QSPLIT) {
            const float2 fl = __half22float2(pl), fh = __half22float2(ph);
            const __half2 ql = __floats2half2_rn(w00 - fl.x, w01 - fl.y), qh = __floats2half2_rn(w10 - fh.x, w11 - fh.y);
            b0l = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ql));
            b1l = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&qh));
        }
    };
    // ---- out^T += V^T . W for the tile at v_tile: MMA j covers coordinates 16j + g (c0, c1) and 16j + g + 8 (c2, c3)
    auto compute_out = [&](int tile, uint32_t v_tile) {
        const int pb = p0 + tile * kTile;
        if (pb + kTile > p1) zero_tail(v_tile, p1 - pb, kSlabsV);
        if constexpr (VB == 2) {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t addr = v_tile + (uint32_t)((j >> 2) * kSlabBytes) + v_row_off + ((((uint32_t)(2 * (j & 3)) + v_csel) ^ key) << 4);
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4_trans(addr, a0, a1, a2, a3);
                mma16816(acc[j], a0, a1, a2, a3, b0, b1);
                if (QSPLIT) mma16816(acc[j], a0, a1, a2, a3, b0l, b1l);
            }
        } else {
            // Block j: coordinates 16 j .. + 15 = 64 bytes of slab j / 2.  Lane (g, t) reads coordinate g (and
            // g + 8) of position rows 2t, 2t + 1, 2t + 8, 2t + 9: 4-byte loads at chunk (4 (j & 1) + g / 4 (+ 2)) ^
            // (row & 7), word g & 3 (rows r and r + 8 share the swizzle).
            const uint32_t ra = (uint32_t)(2 * t), rb = (uint32_t)(2 * t + 1);
            const uint32_t wsel = (uint32_t)((g & 3) * 4);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t slab = v_tile + (uint32_t)((j >> 1) * kSlabBytes) + wsel;
                const uint32_t cl = (uint32_t)(4 * (j & 1) + (g >> 2)), ch = cl + 2;
                const uint32_t a_lo = slab + ra * 128 + ((cl ^ ra) << 4), b_lo = slab + rb * 128 + ((cl ^ rb) << 4);
                const uint32_t a_hi = slab + ra * 128 + ((ch ^ ra) << 4), b_hi = slab + rb * 128 + ((ch ^ rb) << 4);
                float v00, v01, v10, v11, v20, v21, v30, v31;
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v00) : "r"(a_lo));              // dim g,     pos 2t
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v01) : "r"(b_lo));              // dim g,     pos 2t + 1
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v10) : "r"(a_hi));              // dim g + 8, pos 2t
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v11) : "r"(b_hi));              // dim g + 8, pos 2t + 1
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v20) : "r"(a_lo + 8 * 128));    // dim g,     pos 2t + 8
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v21) : "r"(b_lo + 8 * 128));    // dim g,     pos 2t + 9
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v30) : "r"(a_hi + 8 * 128));    // dim g + 8, pos 2t + 8
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v31) : "r"(b_hi + 8 * 128));    // dim g + 8, pos 2t + 9
                uint32_t h0, h1, h2, h3, l0_, l1_, l2_, l3_;
                split_pair(v00, v01, h0, l0_);
                split_pair(v10, v11, h1, l1_);
                split_pair(v20, v21, h2, l2_);
                split_pair(v30, v31, h3, l3_);
                mma16816(acc[j], h0, h1, h2, h3, b0, b1);
                mma16816(acc[j], l0_, l1_, l2_, l3_, b0, b1);
                if (QSPLIT) mma16816(acc[j], h0, h1, h2, h3, b0l, b1l);
            }
        }
    };

    // ---- scan: the warp's tiles are warp, warp + kScanW, ...
    if constexpr (kSplit) {
        // one K and one V buffer per warp; each is refilled with the next tile's half as soon as it is consumed
        uint32_t parity = 0;
        if (warp < kScanW)
            for (int tile = warp; tile < n_tiles; tile += kScanW) {
                const uint32_t st_addr = stage_of(0);
                wait_tile(0, parity);
                compute_scores(tile, st_addr);
                __syncwarp();
                if (tile + kScanW < n_tiles) issue_half(tile + kScanW, 0);
                wait_tile(1, parity);
                compute_out(tile, st_addr + kHalfK);
                __syncwarp();
                if (tile + kScanW < n_tiles) issue_half(tile + kScanW, 1);
                parity ^= 1u;
            }
    } else {
        // tile i lives in stage i % n_stages
        int st = 0;
        uint32_t parity = 0;
        for (int tile = warp; tile < n_tiles; tile += kFW) {
            wait_tile(st, parity);
            compute_scores(tile, stage_of(st));
            compute_out(tile, stage_of(st) + kHalfK);
            __syncwarp();  // every lane has read the stage: lane 0 may refill it
            if (tile + n_stages * kFW < n_tiles) issue_tile(tile + n_stages * kFW, st);
            if (++st == n_stages) { st = 0; parity ^= 1u; }
        }
    }
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // ---- merge the warps (the ring is free now and holds the merge area) ----------------------
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
    __syncthreads();  // every warp has consumed its last stage
    if (tid < 8) {
        float M = -CUDART_INF_F;
        for (int w = 0; w < kFW; w++) M = fmaxf(M, o.m_w[w][tid]);
        float Ls = 0.f;
        for (int w = 0; w < kFW; w++)
            if (o.m_w[w][tid] > -CUDART_INF_F) Ls += o.l_w[w][tid] * exp2f(o.m_w[w][tid] - M);
        o.M[tid] = M;
        o.L[tid] = Ls;
    }
    __syncthreads();
    float *area = reinterpret_cast<float *>(smem_raw + (ring0 - base));  // [kFW][NREP][kHeadStride]
    {
        const float unscale = 1.0f / kWScale;
        const float f0 = (M0 > -CUDART_INF_F) ? exp2f(M0 - o.M[2 * t]) * unscale : 0.f;
        const float f1 = (M1 > -CUDART_INF_F) ? exp2f(M1 - o.M[2 * t + 1]) * unscale : 0.f;
        float *w0 = area + ((size_t)warp * NREP + 2 * t) * kHeadStride + g;
        float *w1 = w0 + kHeadStride;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if (2 * t < NREP) {
                w0[16 * j] = acc[j][0] * f0;
                w0[16 * j + 8] = acc[j][2] * f0;
            }
            if (2 * t + 1 < NREP) {
                w1[16 * j] = acc[j][1] * f1;
                w1[16 * j + 8] = acc[j][3] * f1;
            }
        }
    }
    __syncthreads();
    float sums[NREP];
#pragma unroll
    for (int r = 0; r < NREP; r++) sums[r] = 0.f;
    if (tid < kHd) {
#pragma unroll
        for (int r = 0; r < NREP; r++)
#pragma unroll
            for (int w = 0; w < kFW; w++) sums[r] += area[((size_t)w * NREP + r) * kHeadStride + tid];
    }
    __syncthreads();
    float *s_acc = area;  // [NREP][256]
    if (tid < kHd)
#pragma unroll
        for (int r = 0; r < NREP; r++) s_acc[r * kHd + tid] = sums[r];
    __syncthreads();

    FinishSmem fs;  // the ring behind the merged accumulator carries the streamed combine
    fs.addr = ring0 + (uint32_t)(NREP * kHd * sizeof(float));
    fs.bytes = ring_end - fs.addr;
    fs.bar = base + (uint32_t)offsetof(Other, fin_bar);
    fs.ptr = smem_raw + (fs.addr - base);
    fs.err_flag = err_flag;
    const int first_item = meta.item_start[s] + kv * n_chunks;
    finish_item<NREP, true>(a, meta.slot[s], s, kv, item, n_chunks, first_item, s_acc, o.M, o.L, &o.last, false, nullptr, fs);
}

template <int KB, int VB, int NREP, bool QSPLIT>
bk_status launch_one(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float lut_alpha) {
    using R = Rows<KB, VB>;
    constexpr int kScanW = R::kScanW, kFW = R::kFW, kStageBytes = R::kStageBytes;
    auto *kernel = decode_f16_mma_kernel<KB, VB, NREP, QSPLIT>;
    static std::atomic<size_t> smem_for[64] = {};  // per device; racing first calls compute the same value
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, BK_ERR_UNSUPPORTED, "decode (row mma): device index above 63");
    if (smem_for[dev].load() == 0) {
        cudaFuncAttributes fa;
        BK_CUDA(ctx, cudaFuncGetAttributes(&fa, kernel));
        int optin = 0;
        BK_CUDA(ctx, cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        const size_t dyn = (size_t)optin - fa.sharedSizeBytes;
        // bookkeeping + (planar K) the table + alignment slack + one stage per scanning warp; the merge area must fit the ring
        const size_t need = sizeof(Other) + (R::kPlanarK ? kLutBytes + 256 : 0) + 1024 + (size_t)kScanW * kStageBytes;
        static_assert((size_t)kScanW * kStageBytes >= (size_t)kFW * 6 * kHeadStride * 4, "merge area does not fit the ring");
        if (dyn < need) return fail(ctx, BK_ERR_UNSUPPORTED, "decode (row mma): not enough shared memory per block on this device");
        BK_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
        smem_for[dev].store(dyn);
    }
    const size_t smem = smem_for[dev].load();
    if (!a.h_tmap_k || !a.h_tmap_v) return fail(ctx, BK_ERR_INVALID, "decode (row mma): the cache has no tensor maps");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)m.n_items);
    cfg.blockDim = dim3(R::kFT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol.* in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BK_CUDA(ctx, cudaLaunchKernelEx(&cfg, kernel, a, m, lut_alpha, (uint32_t)smem, ctx->d_err,
                                    *static_cast<const CUtensorMap *>(a.h_tmap_k),
                                    *static_cast<const CUtensorMap *>(a.h_tmap_v)));
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

bool rows_f16(const DecodeArgs &a) { return a.k_kind == ROW_F16 && a.v_kind == ROW_F16 && a.k_row_bytes == 512 && a.v_row_bytes == 512; }
bool rows_f32(const DecodeArgs &a) { return a.k_kind == ROW_F32 && a.v_kind == ROW_F32 && a.k_row_bytes == 1024 && a.v_row_bytes == 1024; }
// K-only planar, 4 or 3 bit: the norms of a tile travel as a 16-byte aligned bulk copy (n_ctx * n_kv a multiple of 4) into a 1 KiB slot
bool rows_pq_f32(const DecodeArgs &a) {
    return a.k_kind == ROW_PLANAR && (a.bits == 4 || a.bits == 3) && a.v_kind == ROW_F32 && a.k_row_bytes == (size_t)(32 * a.bits) &&
           a.v_row_bytes == 1024 && a.seq_stride_rows % 4 == 0 && a.n_kv <= 16;
}

}  // namespace

bool decode_f16_mma_supported(const DecodeArgs &a) {
    const int n_rep = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    return a.h_tmap_k && a.h_tmap_v && (rows_f16(a) || rows_f32(a) || rows_pq_f32(a)) && (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 6);
}

bk_status launch_decode_f16_mma(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float lut_alpha, bool qsplit) {
    if (m.n_items <= 0) return BK_OK;
    const int n_rep = a.n_head / a.n_kv;
    const int kind = rows_f16(a) ? 0 : rows_f32(a) ? 1 : a.bits == 4 ? 2 : 3;
#define BK_F16_CASE(R)                                                                                                            \
    case R:                                                                                                                       \
        if (kind == 2) return qsplit ? launch_one<-4, 4, R, true>(ctx, a, m, lut_alpha) : launch_one<-4, 4, R, false>(ctx, a, m, lut_alpha); \
        if (kind == 3) return qsplit ? launch_one<-3, 4, R, true>(ctx, a, m, lut_alpha) : launch_one<-3, 4, R, false>(ctx, a, m, lut_alpha); \
        if (kind == 1) return qsplit ? launch_one<4, 4, R, true>(ctx, a, m, 1.0f) : launch_one<4, 4, R, false>(ctx, a, m, 1.0f);  \
        return qsplit ? launch_one<2, 2, R, true>(ctx, a, m, 1.0f) : launch_one<2, 2, R, false>(ctx, a, m, 1.0f);
    switch (n_rep) {
        BK_F16_CASE(1)
        BK_F16_CASE(2)
        BK_F16_CASE(4)
        BK_F16_CASE(6)
        default: return fail(ctx, BK_ERR_UNSUPPORTED, "decode (row mma): n_head/n_kv must be 1, 2, 4 or 6");
    }
#undef BK_F16_CASE
}

}  // namespace bk
