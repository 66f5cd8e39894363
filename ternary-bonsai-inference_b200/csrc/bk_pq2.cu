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
//   * the codes go to the tensor cores as they are.  A 32-bit word holds 16 codes; `w & mask`
//     with a two-bit mask in each 16-bit half is a pair of f16 SUBNORMALS of value
//     code * 2^(p-24) (p = the bit position of the code in its half), so one AND makes the A
//     operand of two weights, with no subtraction, table or conversion; five masks on w and
//     three on w >> 6 cover the 16 codes of the word.  The activation that multiplies such a
//     weight is scaled by 2^(15-p) when the CTA stages x (after x is normalised by a power of two
//     so that nothing overflows), which makes every product code * x * 2^-9 exactly;
//   * x is split into f16 hi + lo (22 significant bits) and takes two B columns per token, so
//     m16n8k16 carries up to 4 tokens; the order of the 16 k slots of an MMA is free, and it is
//     chosen so that a lane's A registers come from its own two words of the block;
//   * the "- 1" of the code is the block sum of x, computed once per CTA: per block and row
//     y += scale * (sum x code - sum x), as the reference's scalar path groups it
//     (src/kernels.rs:633-650);
//   * the 8 warps of a CTA split the blocks of a row between them and add up through shared
//     memory.
// The result differs from the reference's scalar path by the summation order and the 22-bit x,
// like its own AVX2 path does (src/kernels.rs:652-660 gives 1e-6 relative for that one).
#include <cuda_fp16.h>
#include <math_constants.h>

#include "bk_device.cuh"
#include "bk_internal.h"
#include "bk_mma_common.cuh"

namespace bk {

namespace {

constexpr int kPqThreads = 256, kPqWarps = 8, kPqTileRows = 16;
constexpr int kPqQK = 128, kPqBlockBytes = 34;
constexpr int kPqMaxStages = 4;

struct Pq2Args {
    const uint8_t *rows;  // first row of the range
    const float *x;       // [n_tok][ne0]
    float *y;             // [n_tok][y_stride]
    int ne0, nb, row_bytes, n_rows, n_tiles, y_stride, n_tok;
    int stages, stage_stride;  // stage_stride: bytes between stages (tile bytes + slack, 128-byte multiple)
    int bulk;                  // 1: tiles start on 16-byte boundaries, the TMA engine may copy them
    int *err_flag;
};

// k-step -> (code index inside a 16-bit half, bit position).  Steps 0-4 mask the word itself,
// steps 5-7 the word shifted right by 6.
__host__ __device__ constexpr int pq_code_of_step(int ks) { return ks < 5 ? 4 - ks : 12 - ks; }
__host__ __device__ constexpr int pq_pos_of_step(int ks) { return ks < 5 ? 8 - 2 * ks : 18 - 2 * ks; }
__host__ __device__ constexpr int pq_step_of_code(int i) { return i < 5 ? 4 - i : 12 - i; }

template <int NT>
__global__ void __launch_bounds__(kPqThreads) pq2_matvec_kernel(const Pq2Args a) {
    extern __shared__ __align__(128) uint8_t sm[];
    constexpr int kCols = 2 * NT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int nb = a.nb;
    // layout: barriers (at 0) | per-token scale | block sums | cross-warp sums | x fragments | stages
    float *inv_s = reinterpret_cast<float *>(sm + 64);
    float *red = reinterpret_cast<float *>(sm + 128);                      // [8 warps][32 lanes][2]
    float *bsum = reinterpret_cast<float *>(sm + 128 + kPqWarps * 32 * 8);  // [NT][nb]
    const uint32_t off_x = (uint32_t)((128 + kPqWarps * 32 * 8 + NT * nb * 4 + 127) / 128 * 128);
    const uint32_t off_st = off_x + (uint32_t)(kCols * nb * 256);
    __half *xf = reinterpret_cast<__half *>(sm + off_x);
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(sm);

    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) mbar_init(sbase + 8u * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    const size_t tile_bytes = (size_t)kPqTileRows * a.row_bytes;
    auto issue = [&](int tile, int st) {  // one thread
        if (!a.bulk || tile >= a.n_tiles || (tile + 1) * kPqTileRows > a.n_rows) return;
        const uint32_t bar = sbase + 8u * st;
        mbar_expect_tx(bar, (uint32_t)tile_bytes);
        tma_bulk(sbase + off_st + (uint32_t)st * a.stage_stride, a.rows + (size_t)tile * tile_bytes, (uint32_t)tile_bytes, bar);
    };
    // The weights do not depend on the kernel before this one: the first copies start at once.
    if (tid == 0)
        for (int s = 0; s < a.stages; s++) issue(blockIdx.x + s * gridDim.x, s);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // ---- x: power-of-two normalisation, block sums, f16 hi/lo fragments ---------------------------
    for (int tok = 0; tok < NT; tok++) {
        const float *xr = a.x + (size_t)tok * a.ne0;
        float am = 0.f;
        const bool real = tok < a.n_tok;  // columns past n_tok are zeros
        for (int j = tid; real && j < a.ne0; j += kPqThreads) am = fmaxf(am, fabsf(xr[j]));
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if (lane == 0) red[warp] = am;
        __syncthreads();
        if (tid == 0) {
            float m = 0.f;
            for (int w = 0; w < kPqWarps; w++) m = fmaxf(m, red[w]);
            int e = 0;
            if (m > 0.f && m < CUDART_INF_F) frexpf(m, &e);  // m = f * 2^e, f in [0.5, 1)
            red[kPqWarps] = ldexpf(1.0f, -e);
            inv_s[tok] = ldexpf(1.0f, e);
        }
        __syncthreads();
        const float s = red[kPqWarps];
        for (int b = warp; b < nb; b += kPqWarps) {
            float part = 0.f;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int jj = lane + 32 * q, j = b * kPqQK + jj;
                const float xv = (real && j < a.ne0) ? xr[j] * s : 0.f;
                part += xv;
                const int tt = jj >> 5, r = (jj >> 4) & 1, e = (jj >> 3) & 1, ks = pq_step_of_code(jj & 7);
                const float xp = xv * (float)(1 << (15 - pq_pos_of_step(ks)));
                const __half hi = __float2half_rn(xp);
                const __half lo = __float2half_rn(xp - __half2float(hi));
                const int base = ((((b * 4 + tt) * 8 + ks) * 2 + r) * 2 + e);
                xf[(size_t)(2 * tok) * nb * 128 + base] = hi;
                xf[(size_t)(2 * tok + 1) * nb * 128 + base] = lo;
            }
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (lane == 0) bsum[tok * nb + b] = part;
        }
        __syncthreads();
    }
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    uint32_t phase = 0;  // one parity bit per stage
    int it = 0;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, it++) {
        const int st = it % a.stages;
        const uint8_t *stage = sm + off_st + (size_t)st * a.stage_stride;
        const int rows_here = min(kPqTileRows, a.n_rows - tile * kPqTileRows);
        if (a.bulk && rows_here == kPqTileRows) {
            int polls = 0;
            while (!mbar_try_wait(sbase + 8u * st, (phase >> st) & 1u)) {
                if (++polls > kWaitPolls) {  // never expected: leave a mark rather than hang
                    if (lane == 0) atomicExch(a.err_flag, 5);
                    break;
                }
            }
            phase ^= 1u << st;
        } else {  // a ragged last tile or an unaligned payload: ordinary 2-byte loads
            const uint16_t *src = reinterpret_cast<const uint16_t *>(a.rows + (size_t)tile * tile_bytes);
            uint16_t *dst = reinterpret_cast<uint16_t *>(sm + off_st + (size_t)st * a.stage_stride);
            const int n2 = rows_here * a.row_bytes / 2;
            for (int i = tid; i < n2; i += kPqThreads) dst[i] = __ldg(src + i);
            __syncthreads();
        }

        float tot0 = 0.f, tot1 = 0.f;
        for (int b = warp; b < nb; b += kPqWarps) {
            // this lane's two words of the block, for rows g and g + 8
            uint32_t w[2][2];
            float sc[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t o = (uint32_t)(g + 8 * h) * a.row_bytes + (uint32_t)b * kPqBlockBytes;
                sc[h] = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(stage + o)));
                const uint32_t oc = o + 2u + 8u * t, al = oc & ~3u, sh = (oc & 2u) * 8u;
                const uint32_t w0 = *reinterpret_cast<const uint32_t *>(stage + al), w1 = *reinterpret_cast<const uint32_t *>(stage + al + 4),
                               w2 = *reinterpret_cast<const uint32_t *>(stage + al + 8);
                w[h][0] = __funnelshift_r(w0, w1, sh);
                w[h][1] = __funnelshift_r(w1, w2, sh);
            }
            uint4 bx[4] = {};
            if (g < kCols) {
                const uint4 *p = reinterpret_cast<const uint4 *>(sm + off_x + ((size_t)(g * nb + b) * 4 + t) * 64);
                bx[0] = p[0]; bx[1] = p[1]; bx[2] = p[2]; bx[3] = p[3];
            }
            const uint32_t *bw = reinterpret_cast<const uint32_t *>(bx);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                const int p = pq_pos_of_step(ks);
                const uint32_t m = (3u << p) | (3u << (p + 16));
                const int shv = ks < 5 ? 0 : 6;
                mma16816(c, (w[0][0] >> shv) & m, (w[1][0] >> shv) & m, (w[0][1] >> shv) & m, (w[1][1] >> shv) & m, bw[2 * ks], bw[2 * ks + 1]);
            }
            const float sx = t < NT ? bsum[t * nb + b] : 0.f;
            tot0 = fmaf(sc[0], fmaf(512.f, c[0] + c[1], -sx), tot0);
            tot1 = fmaf(sc[1], fmaf(512.f, c[2] + c[3], -sx), tot1);
        }
        red[(warp * 32 + lane) * 2] = tot0;
        red[(warp * 32 + lane) * 2 + 1] = tot1;
        __syncthreads();
        if (tid < kPqTileRows * NT) {
            const int r = tid & 15, tok = tid >> 4;
            const int ln = (r & 7) * 4 + tok, h = r >> 3;
            float sum = 0.f;
#pragma unroll
            for (int wp = 0; wp < kPqWarps; wp++) sum += red[(wp * 32 + ln) * 2 + h];
            if (r < rows_here && tok < a.n_tok) a.y[(size_t)tok * a.y_stride + (size_t)tile * kPqTileRows + r] = sum * inv_s[tok];
        }
        __syncthreads();  // the stage and the sums may be overwritten
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            issue(tile + a.stages * (int)gridDim.x, st);
        }
    }
}

template <int NT>
bk_status launch_nt(bk_ctx *ctx, const Pq2Args &a, int grid, size_t smem) {
    BK_CUDA(ctx, cudaFuncSetAttribute(pq2_matvec_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kPqThreads);
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

// rows: device pointer to row 0 of the range; x [n_tok][ne0]; y [n_tok][y_stride], n_tok 1..4.
bk_status launch_pq2_matvec(bk_ctx *ctx, const uint8_t *rows, int ne0, int n_rows, const float *x, int n_tok, float *y, int y_stride) {
    if (n_rows <= 0 || n_tok <= 0) return BK_OK;
    Pq2Args a{};
    a.rows = rows;
    a.x = x;
    a.y = y;
    a.ne0 = ne0;
    a.nb = (ne0 + kPqQK - 1) / kPqQK;
    a.row_bytes = a.nb * kPqBlockBytes;
    a.n_rows = n_rows;
    a.n_tok = n_tok;
    a.n_tiles = (n_rows + kPqTileRows - 1) / kPqTileRows;
    a.y_stride = y_stride;
    a.err_flag = ctx->d_err;
    const size_t tile_bytes = (size_t)kPqTileRows * a.row_bytes;
    a.stage_stride = (int)((tile_bytes + 16 + 127) / 128 * 128);
    a.bulk = ((uintptr_t)rows % 16 == 0) ? 1 : 0;  // 16 rows are a multiple of 16 bytes whatever ne0
    const int nt = n_tok <= 1 ? 1 : (n_tok == 2 ? 2 : 4);
    const size_t fixed = (size_t)((128 + kPqWarps * 32 * 8 + nt * a.nb * 4 + 127) / 128 * 128) + (size_t)2 * nt * a.nb * 256;
    const size_t limit = 227 * 1024;
    if (fixed + 2 * (size_t)a.stage_stride > limit)
        return fail(ctx, BK_ERR_UNSUPPORTED, "pq2_matvec: rows too long for two shared-memory stages of 16 rows");
    // two CTAs per SM when four stages of each fit, else one CTA with as many stages as fit
    int ctas = 2;
    a.stages = kPqMaxStages;
    if (2 * (fixed + (size_t)kPqMaxStages * a.stage_stride + 1024) > limit + 1024) {
        ctas = 1;
        a.stages = (int)std::min<size_t>(kPqMaxStages, (limit - fixed) / a.stage_stride);
    }
    const size_t smem = fixed + (size_t)a.stages * a.stage_stride;
    const int grid = std::min(a.n_tiles, ctx->n_sms * ctas);
    if (nt == 1) return launch_nt<1>(ctx, a, grid, smem);
    if (nt == 2) return launch_nt<2>(ctx, a, grid, smem);
    return launch_nt<4>(ctx, a, grid, smem);
}

}  // namespace bk
