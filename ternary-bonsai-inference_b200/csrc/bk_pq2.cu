// PQ2_0 ternary matrix-vector product: y[t][r] = sum_j x[t][j] * W[base_row + r][j]
// (src/kernels.rs:265-330 `pq2_matvec_range`, 333-420 `pq2_matmul_n`; row format
// src/kernels.rs:204-229: blocks of 34 bytes = one f16 scale + 128 two-bit codes, least
// significant bits first, weight = (code - 1) * scale).
//
// The weight stream is the cost (0.266 bytes per weight, read once), so the kernel is built to
// keep the instruction count per weight low:
//   * a CTA owns tiles of 16 consecutive rows; a tile is one contiguous byte range of the
//     payload, which the TMA engine copies into a ring of shared-memory stages (one bulk copy
//     per tile, completion on an mbarrier);
//   * the codes go to the integer tensor cores as they are.  A 32-bit word holds 16 codes, four
//     per byte; `w & 0x03030303 << 2m` is four unsigned bytes of value 4^m * code, the A operand
//     of mma.m16n8k32.u8.s8 for four weights, with no shift, table or conversion: 16 ANDs and 4
//     MMAs per lane and block cover two rows x 32 weights;
//   * x becomes fixed point when the CTA stages it: per block of 128, X = round(x * 2^(24-e)) with
//     2^e the power of two above the block's max|x| (2^e then rides on the block's f16 scale); the activation that meets a code in byte slot m is B = X * 4^(3-m), so
//     every product is 64 * code * X, and B is split into four balanced base-256 digits, one B
//     column each (two tokens per MMA).  The order of the 32 k slots of an MMA is free, and it
//     is chosen so that a lane's A registers come from its own two words of the block;
//   * the "- 1" of the code is the per-block digit sum of B, an integer computed once per CTA, so
//     the block sums sum (code - 1) * X are EXACT integers; they turn into floats only to be
//     scaled by the block's f16 scale and added up, as the reference's scalar path groups it
//     (src/kernels.rs:633-650);
//   * the 8 warps of a CTA split the blocks of a row between them and add up through shared
//     memory, where the four digit sums are joined.
// The result differs from the reference's scalar path by the summation order across blocks and
// the 2^-25 (block max|x|) grid of X, less than its own AVX2 path does (src/kernels.rs:652-660).
#include <atomic>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "bk_device.cuh"
#include "bk_internal.h"
#include "bk_mma_common.cuh"

namespace bk {

namespace {

constexpr int kPqGroupThreads = 256, kPqWarps = 8, kPqTileRows = 16;  // a group: 8 warps on one tile
constexpr int kPqMaxGroups = 4, kPqGroupStages = 2, kPqMaxSegs = 4;
constexpr int kPqQK = 128, kPqBlockBytes = 34;
constexpr int kPqRedBytes = kPqMaxGroups * 2 * kPqWarps * kPqTileRows * 2 * 4;  // per group two buffers of [warp][row][token]
constexpr int kPqFrac = 24;                          // X = round(x * 2^(kPqFrac - e))

struct Pq2Args {
    // up to kPqMaxSegs row ranges (of tensors with the same ne0) share x and one launch
    const uint8_t *rows[kPqMaxSegs];  // first row of each range
    float *y[kPqMaxSegs];             // [n_tok][seg_rows]
    int seg_rows[kPqMaxSegs];
    int seg_tile0[kPqMaxSegs + 1];    // first tile of each range in the launch's tile order
    const float *x;                   // [n_tok][ne0]
    int ne0, nb, row_bytes, n_tiles, n_tok;
    int stage_stride;  // bytes between stages (tile bytes + slack, 128-byte multiple)
    int groups;        // groups of 8 warps that stream tiles (the CTA always has kPqMaxGroups of them to stage x)
    int stages;        // stages per group: kPqGroupStages, or 1 for rows so long that two do not fit
    int bulk;                  // bit s: the tiles of range s start on 16-byte boundaries, the TMA engine may copy them
    int *err_flag;
};

// D (s32) += A (u8, 16 x 32, row) . B (s8, 32 x 8, col).  No side effects: the compiler may schedule it.
__device__ __forceinline__ void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared memory: barriers (at 0) | partial sums (at 256) | digit sums [nb][8] | block scales [2][nb] | x digits | stages
__host__ __device__ inline uint32_t pq_off_dsum() { return 256u + kPqRedBytes; }
__host__ __device__ inline uint32_t pq_off_x(int nb) { return (pq_off_dsum() + (uint32_t)nb * 40u + 127u) / 128u * 128u; }
__host__ __device__ inline uint32_t pq_off_stage(int nb, int nt) { return pq_off_x(nb) + (uint32_t)(4 * nt) * nb * 128u; }

template <int NT>
__global__ void __launch_bounds__(kPqGroupThreads * kPqMaxGroups) pq2_matvec_kernel(const Pq2Args a) {
    extern __shared__ __align__(128) uint8_t sm[];
    constexpr int kCols = 4 * NT;  // four base-256 digits per token
    // all threads stage x; then every group of 8 warps streams its own tiles through its own stages
    const int tid_all = threadIdx.x, warp_all = tid_all >> 5, n_threads = blockDim.x, n_warps = n_threads >> 5, n_groups = a.groups;
    const int grp = warp_all / kPqWarps, warp = warp_all % kPqWarps, tid = tid_all % kPqGroupThreads;
    const int lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int nb = a.nb;
    float *red = reinterpret_cast<float *>(sm + 256);
    int *dsum = reinterpret_cast<int *>(sm + pq_off_dsum());
    float *bscale = reinterpret_cast<float *>(sm + pq_off_dsum() + (uint32_t)nb * 32u);  // [2][nb]
    const uint32_t off_x = pq_off_x(nb), off_st = pq_off_stage(nb, NT);
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(sm);

    if (tid_all == 0) {
        for (int s = 0; s < kPqMaxGroups * kPqGroupStages; s++) mbar_init(sbase + 8u * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    for (int i = tid_all; i < nb * 8; i += n_threads) dsum[i] = 0;
    __syncthreads();

    const size_t tile_bytes = (size_t)kPqTileRows * a.row_bytes;
    auto seg_of = [&](int tile) {
        int sg = 0;
#pragma unroll
        for (int i = 1; i < kPqMaxSegs; i++) sg += (tile >= a.seg_tile0[i]) ? 1 : 0;  // unused ranges start at n_tiles
        return sg;
    };
    // the it-th tile of this group: consecutive CTAs take consecutive tiles, group after group, so a last
    // partial round spreads over all SMs (few groups busy on each) instead of filling some of them
    auto tile_of = [&](int it) { return (it * n_groups + grp) * (int)gridDim.x + (int)blockIdx.x; };
    auto issue = [&](int it) {  // one thread of the group
        const int tile = tile_of(it), st = grp * a.stages + it % a.stages;
        if (tile >= a.n_tiles) return;
        const int sg = seg_of(tile), lt = tile - a.seg_tile0[sg];
        if (!((a.bulk >> sg) & 1) || (lt + 1) * kPqTileRows > a.seg_rows[sg]) return;
        const uint32_t bar = sbase + 8u * st;
        mbar_expect_tx(bar, (uint32_t)tile_bytes);
        tma_bulk(sbase + off_st + (uint32_t)st * a.stage_stride, a.rows[sg] + (size_t)lt * tile_bytes, (uint32_t)tile_bytes, bar);
    };
    // The weights do not depend on the kernel before this one: the first copies start at once.
    if (tid == 0 && grp < n_groups)
        for (int s = 0; s < a.stages; s++) issue(s);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // ---- x: per block a power-of-two scale, fixed point, balanced digits, digit sums --------------
    // One warp per (token, block): X = round(x * 2^(24 - e)) with 2^e the power of two above the
    // block's max |x|; the block's 2^(e - 24 - 6) (the products carry 4^3) multiplies its f16 scale.
    // Element jj of a block (32 t + 16 r + 4 q + m: word 2t + r of the block, byte q, slot m) lands in
    // byte q of the word [col][block][t][m][r]; a lane's 8 words of a block are 32 contiguous bytes.
    for (int unit = warp_all; unit < NT * nb; unit += n_warps) {
        const int tok = unit / nb, b = unit - tok * nb;
        const float *xr = a.x + (size_t)tok * a.ne0;
        const bool real = tok < a.n_tok;  // columns past n_tok are zeros
        float xv[4], am = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int j = b * kPqQK + lane + 32 * i;
            xv[i] = (real && j < a.ne0) ? xr[j] : 0.f;
            am = fmaxf(am, fabsf(xv[i]));
        }
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        int e = 0;
        if (am > 0.f && am < CUDART_INF_F) frexpf(am, &e);  // am = f * 2^e, f in [0.5, 1)
        const float s = ldexpf(1.0f, kPqFrac - e);
        int ds[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int jj = lane + 32 * i;
            const int tt = jj >> 5, r = (jj >> 4) & 1, q = (jj >> 2) & 3, m = jj & 3;
            int B = __float2int_rn(xv[i] * s) << (2 * (3 - m));  // |x s| < 2^24
            uint8_t *dst = sm + off_x + ((((size_t)(4 * tok) * nb + b) * 4 + tt) * 8 + m * 2 + r) * 4 + q;
#pragma unroll
            for (int d = 0; d < 4; d++) {
                const int dg = (int)(int8_t)(B & 0xff);
                B = (B - dg) >> 8;
                dst[(size_t)d * nb * 128] = (uint8_t)dg;
                ds[d] += dg << (2 * m);
            }
        }
#pragma unroll
        for (int d = 0; d < 4; d++) {
            int v = ds[d];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) dsum[b * 8 + 4 * tok + d] = v;
        }
        if (lane == 0) bscale[tok * nb + b] = ldexpf(1.0f, e - kPqFrac - 6);
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // per-lane constants of the weight reads: rows g and g + 8, this lane's 8 bytes of a block
    uint32_t w_off[2], w_sh[2], s_off[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        s_off[h] = (uint32_t)(g + 8 * h) * a.row_bytes + (uint32_t)warp * kPqBlockBytes;
        const uint32_t oc = s_off[h] + 2u + 8u * t;
        w_off[h] = oc & ~3u;         // the warp's next block is 8 * 34 = 272 bytes on: the alignment stays
        w_sh[h] = (oc & 2u) * 8u;
    }
    const bool has_x = g < kCols;
    const uint32_t x_lane = off_x + ((uint32_t)(g * nb + warp) * 4 + t) * 32;
    const uint32_t d_lane = pq_off_dsum() + (uint32_t)warp * 32 + 8u * t;
    const uint32_t bs_lane = pq_off_dsum() + (uint32_t)nb * 32u + (uint32_t)((t >> 1) * nb + warp) * 4u;

    if (grp >= n_groups) return;  // helped to stage x; no tiles for this group
    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;\n" ::"r"(1 + grp), "r"(kPqGroupThreads) : "memory"); };
    float *red_g = red + grp * (2 * kPqWarps * kPqTileRows * 2);
    uint32_t phase = 0;  // one parity bit per stage of the group
    for (int it = 0;; it++) {
        const int tile = tile_of(it);
        if (tile >= a.n_tiles) break;
        const int sl = it % a.stages, st = grp * a.stages + sl;
        const uint8_t *stage = sm + off_st + (size_t)st * a.stage_stride;
        const int sg = seg_of(tile), lt = tile - a.seg_tile0[sg];
        const int rows_here = min(kPqTileRows, a.seg_rows[sg] - lt * kPqTileRows);
        if (((a.bulk >> sg) & 1) && rows_here == kPqTileRows) {
            int polls = 0;
            while (!mbar_try_wait(sbase + 8u * st, (phase >> sl) & 1u)) {
                if (++polls > kWaitPolls) {  // never expected: leave a mark rather than hang
                    if (lane == 0) raise_error(a.err_flag, 5);
                    break;
                }
            }
            phase ^= 1u << sl;
        } else {  // a ragged last tile or an unaligned payload: ordinary 2-byte loads
            const uint16_t *src = reinterpret_cast<const uint16_t *>(a.rows[sg] + (size_t)lt * tile_bytes);
            uint16_t *dst = reinterpret_cast<uint16_t *>(sm + off_st + (size_t)st * a.stage_stride);
            const int n2 = rows_here * a.row_bytes / 2;
            for (int i = tid; i < n2; i += kPqGroupThreads) dst[i] = __ldg(src + i);
            group_sync();
        }

        float tot[4] = {0.f, 0.f, 0.f, 0.f};  // rows g (0, 1) and g + 8 (2, 3), digit columns 2t and 2t + 1
        uint32_t step = 0;
#pragma unroll 2
        for (int b = warp; b < nb; b += kPqWarps, step += 1) {
            uint32_t w[2][2];
            float sc[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint8_t *pw = stage + w_off[h] + step * (kPqWarps * kPqBlockBytes);
                const uint32_t w0 = *reinterpret_cast<const uint32_t *>(pw), w1 = *reinterpret_cast<const uint32_t *>(pw + 4),
                               w2 = *reinterpret_cast<const uint32_t *>(pw + 8);
                w[h][0] = __funnelshift_r(w0, w1, w_sh[h]);
                w[h][1] = __funnelshift_r(w1, w2, w_sh[h]);
                sc[h] = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(stage + s_off[h] + step * (kPqWarps * kPqBlockBytes))));
            }
            uint4 bx0 = make_uint4(0, 0, 0, 0), bx1 = bx0;
            if (has_x) {
                const uint4 *px = reinterpret_cast<const uint4 *>(sm + x_lane + step * (kPqWarps * 128));
                bx0 = px[0];
                bx1 = px[1];
            }
            const int2 dsv = *reinterpret_cast<const int2 *>(sm + d_lane + step * (kPqWarps * 32));
            const float bs = *reinterpret_cast<const float *>(sm + bs_lane + step * (kPqWarps * 4));
            sc[0] *= bs;
            sc[1] *= bs;
            int c[4] = {-dsv.x, -dsv.y, -dsv.x, -dsv.y}, c2[4] = {0, 0, 0, 0};  // two chains; the "- 1" goes in as the start value
            imma_u8s8(c, w[0][0] & 0x03030303u, w[1][0] & 0x03030303u, w[0][1] & 0x03030303u, w[1][1] & 0x03030303u, bx0.x, bx0.y);
            imma_u8s8(c2, w[0][0] & 0x0c0c0c0cu, w[1][0] & 0x0c0c0c0cu, w[0][1] & 0x0c0c0c0cu, w[1][1] & 0x0c0c0c0cu, bx0.z, bx0.w);
            imma_u8s8(c, w[0][0] & 0x30303030u, w[1][0] & 0x30303030u, w[0][1] & 0x30303030u, w[1][1] & 0x30303030u, bx1.x, bx1.y);
            imma_u8s8(c2, w[0][0] & 0xc0c0c0c0u, w[1][0] & 0xc0c0c0c0u, w[0][1] & 0xc0c0c0c0u, w[1][1] & 0xc0c0c0c0u, bx1.z, bx1.w);
            tot[0] = fmaf(sc[0], (float)(c[0] + c2[0]), tot[0]);
            tot[1] = fmaf(sc[0], (float)(c[1] + c2[1]), tot[1]);
            tot[2] = fmaf(sc[1], (float)(c[2] + c2[2]), tot[2]);
            tot[3] = fmaf(sc[1], (float)(c[3] + c2[3]), tot[3]);
        }
        // join the four digits: this lane's two columns, then the lane pair (t even: digits 0 1, t odd: 2 3)
        float v0 = fmaf(tot[1], 256.f, tot[0]), v1 = fmaf(tot[3], 256.f, tot[2]);
        v0 = fmaf(__shfl_xor_sync(0xffffffffu, v0, 1), 65536.f, v0);  // meaningful on even t only
        v1 = fmaf(__shfl_xor_sync(0xffffffffu, v1, 1), 65536.f, v1);
        float *rd = red_g + (it & 1) * (kPqWarps * kPqTileRows * 2);  // [warp][row][token]; two buffers: one barrier per tile
        if ((t & 1) == 0 && (t >> 1) < NT) {
            rd[(warp * kPqTileRows + g) * 2 + (t >> 1)] = v0;
            rd[(warp * kPqTileRows + g + 8) * 2 + (t >> 1)] = v1;
        }
        group_sync();  // the tile's partial sums are in place, and nobody of the group reads the stage any more
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            issue(it + a.stages);
        }
        if (tid < kPqTileRows * NT) {
            const int r = tid & 15, tok = tid >> 4;
            float sum = 0.f;
#pragma unroll
            for (int wp = 0; wp < kPqWarps; wp++) sum += rd[(wp * kPqTileRows + r) * 2 + tok];
            if (r < rows_here && tok < a.n_tok) a.y[sg][(size_t)tok * a.seg_rows[sg] + (size_t)lt * kPqTileRows + r] = sum;
        }
    }
}

template <int NT>
bk_status launch_nt(bk_ctx *ctx, const Pq2Args &a, int grid, size_t smem) {
    static std::atomic<bool> opted_in[64] = {};  // the opt-in is per device and costs a driver call: once per device is enough
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, BK_ERR_UNSUPPORTED, "pq2 matvec: device index above 63");
    if (!opted_in[dev].load()) {
        BK_CUDA(ctx, cudaFuncSetAttribute(pq2_matvec_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        opted_in[dev].store(true);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)(kPqGroupThreads * kPqMaxGroups));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BK_CUDA(ctx, cudaLaunchKernelEx(&cfg, pq2_matvec_kernel<NT>, a));
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace

size_t pq2_row_bytes(int64_t ne0) { return (size_t)((ne0 + kPqQK - 1) / kPqQK) * kPqBlockBytes; }

// Up to four row ranges with the same ne0 (rows[s]: device pointer to the first row, n_rows[s] rows,
// y[s] [n_tok][n_rows[s]]); x [n_tok][ne0], n_tok 1..2.
bk_status launch_pq2_matvec(bk_ctx *ctx, int n_seg, const uint8_t *const *rows, const int *n_rows, float *const *y, int ne0,
                            const float *x, int n_tok) {
    if (n_tok <= 0) return BK_OK;
    Pq2Args a{};
    a.x = x;
    a.ne0 = ne0;
    a.nb = (ne0 + kPqQK - 1) / kPqQK;
    a.row_bytes = a.nb * kPqBlockBytes;
    a.n_tok = n_tok;
    a.err_flag = ctx->d_err;
    int tiles = 0, used = 0;
    for (int sgi = 0; sgi < n_seg && used < kPqMaxSegs; sgi++) {
        if (n_rows[sgi] <= 0) continue;
        a.rows[used] = rows[sgi];
        a.y[used] = y[sgi];
        a.seg_rows[used] = n_rows[sgi];
        a.seg_tile0[used] = tiles;
        if ((uintptr_t)rows[sgi] % 16 == 0) a.bulk |= 1 << used;  // 16 rows are a multiple of 16 bytes whatever ne0
        tiles += (n_rows[sgi] + kPqTileRows - 1) / kPqTileRows;
        used++;
    }
    for (int sgi = used; sgi <= kPqMaxSegs; sgi++) a.seg_tile0[sgi] = tiles;
    a.n_tiles = tiles;
    if (tiles == 0) return BK_OK;
    const size_t tile_bytes = (size_t)kPqTileRows * a.row_bytes;
    a.stage_stride = (int)((tile_bytes + 16 + 127) / 128 * 128);
    const int nt = n_tok <= 1 ? 1 : 2;
    const size_t fixed = pq_off_stage(a.nb, nt);
    const size_t limit = 227 * 1024;
    a.stages = fixed + (size_t)kPqGroupStages * a.stage_stride <= limit ? kPqGroupStages : 1;
    const size_t per_group = (size_t)a.stages * a.stage_stride;
    if (fixed + per_group > limit)
        return fail(ctx, BK_ERR_UNSUPPORTED, "pq2_matvec: rows too long for a shared-memory stage of 16 rows");
    // One CTA per SM; it runs as many groups of 8 warps (each with its own tiles and stages) as the
    // matrix has tiles for and shared memory has room for.
    int groups = (int)std::min<size_t>(kPqMaxGroups, (limit - fixed) / per_group);
    groups = std::max(1, std::min(groups, (a.n_tiles + ctx->n_sms - 1) / ctx->n_sms));
    a.groups = groups;
    const size_t smem = fixed + (size_t)groups * per_group;
    const int grid = std::min(a.n_tiles, ctx->n_sms);
    if (nt == 1) return launch_nt<1>(ctx, a, grid, smem);
    return launch_nt<2>(ctx, a, grid, smem);
}

}  // namespace bk
