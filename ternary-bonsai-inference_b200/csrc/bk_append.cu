// Fused KV append: IMROPE on K, then store K and V rows as f32, f16 or rotated Lloyd-Max
// ("planar") rows, one launch for any number of tokens.  Replaces rope_imrope.comp (k side),
// kv_store.comp, kv_store_f16.comp and kv_store_q.comp and follows the reference CPU path
// bit for bit (src/forward.rs:259-285, src/kvquant.rs:397-412, src/rope.rs:61-69).
//
// A CTA stages 32 vectors of 256 floats ((K|V, kv head) of consecutive tokens):
//   1. coalesced float4 loads into shared memory; K vectors rotate pairs (j, j + n_rot/2) with
//      the (cos, sin) row of the token's position from the host-built rope table;
//   2. planar rows: one warp adds the 256 squares of all 32 vectors, a vector per lane, each lane
//      in order (the reference's f32 sum is sequential, so each chain is; 32 run side by side);
//   3. the warps scale, Givens-rotate, find the nearest centroid (a cell table or a binary search, then
//      one neighbour check: the same index as the reference's linear scan) and write `bits` bytes per lane;
//      f32/f16 rows leave as 128-bit stores.
// Traffic per token is the algorithmic minimum: 2*n_kv*1 KiB in, rows + norms out.
#include "bk_device.cuh"
#include "bk_internal.h"

namespace bk {

namespace {

constexpr int kVecPad = kHd + 4;  // floats per staged vector; +4 keeps float4 alignment and makes the
                                  // per-lane 128-bit reads of the norm pass conflict-free
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

// Rotate, quantize and pack the 8 coordinates of one lane; `n` is the vector's norm.
template <int BITS>
__device__ __forceinline__ void store_planar_row(const float *sx, int lane, float n, const float *givens,
                                                 const float *sbook, uint8_t *row) {
    const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
    uint64_t packed = 0;
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        const int i = lane * 4 + pr;  // pair index: coordinates 2i, 2i+1
        const float a = __fmul_rn(sx[2 * i], inv), b = __fmul_rn(sx[2 * i + 1], inv);
        float r0, r1;
        givens_fwd(a, b, givens[2 * i], givens[2 * i + 1], r0, r1);
        packed |= (uint64_t)nearest_centroid_fast<BITS>(r0, sbook) << (BITS * (2 * pr));
        packed |= (uint64_t)nearest_centroid_fast<BITS>(r1, sbook) << (BITS * (2 * pr + 1));
    }
    store_group8<BITS>(row, lane, packed);
}

// The same with the two-read centroid search (codebooks of up to 16 centroids).
template <int BITS>
__device__ __forceinline__ void store_planar_row_cell(const float *sx, int lane, float n, const float *givens,
                                                      const float *sbook, const float4 *b4, const uint8_t *cells, uint8_t *row) {
    const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
    uint64_t packed = 0;
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        const int i = lane * 4 + pr;  // pair index: coordinates 2i, 2i+1
        const float a = __fmul_rn(sx[2 * i], inv), b = __fmul_rn(sx[2 * i + 1], inv);
        float r0, r1;
        givens_fwd(a, b, givens[2 * i], givens[2 * i + 1], r0, r1);
        packed |= (uint64_t)nearest_centroid_cell<BITS>(r0, sbook, b4, cells) << (BITS * (2 * pr));
        packed |= (uint64_t)nearest_centroid_cell<BITS>(r1, sbook, b4, cells) << (BITS * (2 * pr + 1));
    }
    store_group8<BITS>(row, lane, packed);
}

__device__ __forceinline__ void store_f32_row(const float *sx, int lane, uint8_t *row) {
    float4 *dst = reinterpret_cast<float4 *>(row);
    const float4 *src = reinterpret_cast<const float4 *>(sx);
    dst[lane] = src[lane];
    dst[lane + 32] = src[lane + 32];
}

__device__ __forceinline__ void store_f16_row(const float *sx, int lane, uint8_t *row) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t lo = f32_to_half_ref(sx[lane * 8 + 2 * i]);
        const uint32_t hi = f32_to_half_ref(sx[lane * 8 + 2 * i + 1]);
        w[i] = lo | (hi << 16);
    }
    reinterpret_cast<uint4 *>(row)[lane] = make_uint4(w[0], w[1], w[2], w[3]);
}

// A CTA takes 32 consecutive vectors of the launch (vector = token * 2*n_kv + j; j < n_kv: K head
// j, else V head j - n_kv).  Pass 1: each warp stages 8 vectors with float4 loads and ropes the K
// ones.  Pass 2: warp 0 adds the squares of all 32 vectors, one vector per lane, each lane in
// order (the reference's f32 sum is sequential, so the chain is; 32 chains run side by side).
// Pass 3: each warp scales, rotates, finds the nearest centroids of and stores its 8 vectors.
// kVecs = 32 for bulk calls (throughput: every lane of the norm pass works), 8 for small calls
// (latency: one vector per warp).
template <int BITS, int kVecs>
__global__ void __launch_bounds__(kThreads) append_kernel(AppendArgs a) {
    extern __shared__ __align__(16) float smem[];
    float *sbook = smem + kVecs * kVecPad;  // centroids
    float *sgiv = sbook + 256;              // Givens table
    float *snorm = sgiv + kHd;              // the 32 norms
    [[maybe_unused]] float4 *b4 = reinterpret_cast<float4 *>(snorm + 32);   // centroid neighbourhoods of the two-read search
    [[maybe_unused]] uint8_t *cells = reinterpret_cast<uint8_t *>(b4 + 16); // its 512 cells
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kv = a.n_kv, per_tok = 2 * n_kv;
    const int n_vec = a.n_tokens * per_tok, v0 = blockIdx.x * kVecs;
    const bool planar = a.k_kind == ROW_PLANAR || a.v_kind == ROW_PLANAR;

    if (BITS > 0) {
        for (int i = threadIdx.x; i < (1 << BITS); i += kThreads) sbook[i] = a.book[i];
        for (int i = threadIdx.x; i < kHd; i += kThreads) sgiv[i] = a.givens[i];
        if constexpr (BITS >= 1 && BITS <= 4) {
            __syncthreads();
            build_cell_tables(sbook, 1 << BITS, b4, cells);
        }
    }
    // k and v may come from the previous kernel in the stream: with programmatic dependent launch
    // only the table copies above run ahead of it.  Nothing after this kernel depends on more
    // than its completion, so dependents may be scheduled right away.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // ---- pass 1: stage (and rope).  A warp owns vectors warp, warp + 8, ...; all of their global
    // loads (rows and rope entries) are issued before any is used, so the pass costs one round trip.
    constexpr int kPerWarp = kVecs / kWarps;
    float4 ra[kPerWarp], rb[kPerWarp];
    float2 rcs[kPerWarp];
    const int half = a.n_rot >> 1;
#pragma unroll
    for (int u = 0; u < kPerWarp; u++) {
        const int vec = v0 + warp + u * kWarps;
        ra[u] = rb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        rcs[u] = make_float2(1.f, 0.f);
        if (vec < n_vec) {
            const int tok = vec / per_tok, j = vec - tok * per_tok;
            const bool is_v = j >= n_kv;
            const int kv = is_v ? j - n_kv : j;
            const float4 *src4 = reinterpret_cast<const float4 *>((is_v ? a.v : a.k) + ((size_t)tok * n_kv + kv) * kHd);
            ra[u] = __ldg(src4 + lane);
            rb[u] = __ldg(src4 + lane + 32);
            if (!is_v && lane < half) {  // n_rot <= 64: one rope entry per lane
                const int pos = a.desc ? a.desc[tok].z : a.pos0 + tok;
                rcs[u] = __ldg(a.rope + (size_t)pos * half + lane);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kPerWarp; u++) {
        const int lv = warp + u * kWarps, vec = v0 + lv;
        if (vec >= n_vec) continue;
        float *sx = smem + lv * kVecPad;
        reinterpret_cast<float4 *>(sx)[lane] = ra[u];
        reinterpret_cast<float4 *>(sx)[lane + 32] = rb[u];
        const bool is_v = (vec % per_tok) >= n_kv;
        if (!is_v) {
            __syncwarp();
            if (half <= 32) {
                if (lane < half) {
                    float x0 = sx[lane], x1 = sx[lane + half];
                    rope_pair(x0, x1, rcs[u]);
                    sx[lane] = x0;
                    sx[lane + half] = x1;
                }
            } else {  // wider rotations: entries beyond the prefetched 32 come straight from the table
                const int tok = vec / per_tok, pos = a.desc ? a.desc[tok].z : a.pos0 + tok;
                const float2 *cs = a.rope + (size_t)pos * half;
                for (int p = lane; p < half; p += 32) {
                    float x0 = sx[p], x1 = sx[p + half];
                    rope_pair(x0, x1, cs[p]);
                    sx[p] = x0;
                    sx[p + half] = x1;
                }
            }
        }
    }
    __syncthreads();
    // ---- pass 2: 32 sequential sums side by side ----------------------------------------------------
    if (planar && warp == 0 && lane < kVecs && v0 + lane < n_vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(smem + lane * kVecPad);
        float acc = 0.0f;
#pragma unroll 8
        for (int i = 0; i < kHd / 4; i++) {
            const float4 x = x4[i];
            acc = __fadd_rn(acc, __fmul_rn(x.x, x.x));
            acc = __fadd_rn(acc, __fmul_rn(x.y, x.y));
            acc = __fadd_rn(acc, __fmul_rn(x.z, x.z));
            acc = __fadd_rn(acc, __fmul_rn(x.w, x.w));
        }
        snorm[lane] = __fsqrt_rn(acc);
    }
    __syncthreads();
    // ---- pass 3: store --------------------------------------------------------------------------------
    for (int lv = warp; lv < kVecs; lv += kWarps) {
        const int vec = v0 + lv;
        if (vec >= n_vec) break;
        const int tok = vec / per_tok, j = vec - tok * per_tok;
        const bool is_v = j >= n_kv;
        const int kv = is_v ? j - n_kv : j;
        size_t seq_rows = 0;
        int row_idx;
        if (a.desc) {
            const int4 d = a.desc[tok];
            seq_rows = (size_t)d.x * a.seq_stride_rows;
            row_idx = d.y;
        } else {
            row_idx = a.row0 + tok;
        }
        const float *sx = smem + lv * kVecPad;
        const size_t r = seq_rows + (size_t)row_idx * n_kv + kv;
        const int kind = is_v ? a.v_kind : a.k_kind;
        uint8_t *row = (is_v ? a.v_rows + r * a.v_row_bytes : a.k_rows + r * a.k_row_bytes);
        if (kind == ROW_F32) {
            store_f32_row(sx, lane, row);
        } else if (kind == ROW_F16) {
            store_f16_row(sx, lane, row);
        } else {
            if constexpr (BITS > 0) {
                const float n = snorm[lv];
                if (lane == 0) (is_v ? a.v_norms : a.k_norms)[r] = n;
                if constexpr (BITS <= 4) store_planar_row_cell<BITS>(sx, lane, n, sgiv, sbook, b4, cells, row);
                else store_planar_row<BITS>(sx, lane, n, sgiv, sbook, row);
            }
        }
    }
}


}  // namespace

bk_status launch_append(bk_ctx *ctx, const AppendArgs &a) {
    if (a.n_tokens <= 0) return BK_OK;
    const int threads = kThreads;
    const size_t n_vec = (size_t)a.n_tokens * 2 * a.n_kv;
    const bool bulk = n_vec > (size_t)8 * 2 * ctx->n_sms;  // more than two small CTAs per SM: go for throughput
    const int vecs = bulk ? 32 : 8;
    const size_t smem = (size_t)(vecs * kVecPad + 256 + kHd + 32) * sizeof(float) + 16 * sizeof(float4) + 512;
    const unsigned grid = (unsigned)((n_vec + vecs - 1) / vecs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol.* in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaSuccess;
    const bool planar = a.k_kind == ROW_PLANAR || a.v_kind == ROW_PLANAR;
    if (!planar) {
        err = bulk ? cudaLaunchKernelEx(&cfg, append_kernel<0, 32>, a) : cudaLaunchKernelEx(&cfg, append_kernel<0, 8>, a);
    } else {
        const bool ok = dispatch_bits(a.bits, [&]<int B>() {
            err = bulk ? cudaLaunchKernelEx(&cfg, append_kernel<B, 32>, a) : cudaLaunchKernelEx(&cfg, append_kernel<B, 8>, a);
        });
        if (!ok) return fail(ctx, BK_ERR_INVALID, "append: bits must be 1..8");
    }
    ctx->launches++;
    BK_CUDA(ctx, err);
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace bk
